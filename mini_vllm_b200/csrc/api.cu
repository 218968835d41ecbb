// Version and status strings of the C ABI, and the self-test of the bounded device wait.
#include "common.cuh"
#include "mini_vllm_b200.h"

extern "C" int mvb_abi_version(void) { return 6; }

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

namespace mvb {

// One warp waits, with the same bounded mbar_wait the attention kernels use, on a barrier that nobody
// will ever arrive at.  The wait runs out after `limit` polls, the kernel records kDevWaitTimeout in the
// status word and returns normally: the context stays usable.
__global__ void selftest_wait_kernel(int* dev_status, uint32_t limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  const bool ok = mbar_wait(&bar, 0, limit);
  if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) report(dev_status, kDevWaitTimeout, static_cast<int>(limit));
}

}  // namespace mvb

extern "C" int mvb_selftest_wait_timeout(int32_t* dev_status, int limit, void* stream) {
  if (dev_status == nullptr || limit <= 0 || limit > (1 << 16)) return mvb::kInvalidArgument;
  mvb::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev_status, static_cast<uint32_t>(limit));
  return cudaGetLastError() == cudaSuccess ? mvb::kOk : mvb::kLaunchFailed;
}
