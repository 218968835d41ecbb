// Host-side helpers shared by the entry points: tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda), device properties, alignment checks.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "common.cuh"

namespace mvb {

inline bool is_aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// bf16 tensor viewed as [rows, heads, head_dim] (head_dim innermost, contiguous heads, free row
// stride); box = (64 elements, 1 head, box_rows rows), 128-byte swizzle.  Out-of-range rows read
// as zeros.
inline int make_kv_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int heads, int head_dim,
                              int64_t row_stride_elems, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return kNoDriverEntry;
  if (!is_aligned(base, 16) || (row_stride_elems % 8) != 0 || head_dim % 64 != 0) return kMisaligned;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(row_stride_elems) * 2};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kTensorMapFailed;
}

// Per-device facts are looked up once per device, under a lock, so that the first calls of two threads
// (or calls on two different GPUs of one process) cannot see each other's half-written state.
constexpr int kMaxDevices = 64;

inline int sm_count() {
  static std::mutex mu;
  static int by_device[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (by_device[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    by_device[dev] = v;
  }
  return by_device[dev];
}

// Opts a kernel in to `bytes` of dynamic shared memory (beyond the 48 KB default) once per device and
// size.  Tag names the kernel instantiation: each one keeps its own table.
template <class Tag>
inline int opt_in_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static size_t configured[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kLaunchFailed;
  std::lock_guard<std::mutex> lock(mu);
  if (bytes > configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
      return kLaunchFailed;
    configured[dev] = bytes;
  }
  return kOk;
}

}  // namespace mvb
