// Block-wide exclusive prefix sum used by the packing and planning kernels.
#pragma once
#include <stdint.h>

namespace mvb {

// Exclusive prefix sum of f(i), i in [0,n), into out[0..n] (out[n] = total).  out may be shared
// or global memory.  Must be called by all THREADS threads of the block (THREADS % 32 == 0).
template <int THREADS, class F>
__device__ void block_exclusive_scan(F f, int n, int32_t* out) {
  __shared__ int32_t warp_tot[THREADS / 32];
  __shared__ int32_t carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n; base += THREADS) {
    const int i = base + tid;
    const int32_t v = i < n ? f(i) : 0;
    int32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int32_t off = carry_s;
    for (int w = 0; w < warp; ++w) off += warp_tot[w];
    if (i < n) out[i] = off + inc - v;
    __syncthreads();
    if (tid == THREADS - 1) carry_s = off + inc;
    __syncthreads();
  }
  if (tid == 0) out[n] = carry_s;
  __syncthreads();
}

}  // namespace mvb
