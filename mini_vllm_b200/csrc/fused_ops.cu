// Glue kernels of the decoder layer around the attention path.  A decode step of a small model is
// bound by the NUMBER of kernels (a few microseconds each, whatever their size), so the elementwise
// chains between the GEMMs are fused: activation * up-projection, and residual add + RMSNorm
// (optionally with Gemma's extra norm on the branch output).  Each intermediate is rounded to bf16
// where the unfused PyTorch sequence would round it, so results match that sequence to an ulp.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

namespace mvb {

// SiLU as x * sigmoid(x) through the fast exponential and a correctly rounded reciprocal: a few fp32 ulps from
// x / (1 + expf(-x)), far below the bf16 rounding that follows, at a third of the instructions (with the library
// forms the kernel is bound by its instruction count, not by memory).  The tanh-GELU keeps the library tanhf:
// in its negative tail 1 + tanh(u) cancels, and only the same form rounds there like the eager sequence.
__device__ __forceinline__ float act_silu(float x) { return x * __frcp_rn(1.f + __expf(-x)); }
__device__ __forceinline__ float act_gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]
// blockIdx.x picks the 16-byte chunk of the row, blockIdx.y the first of the rows the thread walks (two at a
// time, so four loads are in flight per thread); no index arithmetic beyond adds.
constexpr int kActThreads = 128;

__device__ __forceinline__ uint4 act_mul8(const uint4& gv, const uint4& uv, int gelu) {
  const uint32_t* ga = reinterpret_cast<const uint32_t*>(&gv);
  const uint32_t* ua = reinterpret_cast<const uint32_t*>(&uv);
  uint4 ov;
  uint32_t* oa = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float g0 = bf16_lo(ga[i]), g1 = bf16_hi(ga[i]);
    const float a0 = round_bf16(gelu ? act_gelu_tanh(g0) : act_silu(g0));
    const float a1 = round_bf16(gelu ? act_gelu_tanh(g1) : act_silu(g1));
    oa[i] = pack_bf16(a0 * bf16_lo(ua[i]), a1 * bf16_hi(ua[i]));
  }
  return ov;
}

__global__ void __launch_bounds__(kActThreads) act_mul_kernel(const __nv_bfloat16* __restrict__ gate_up, int64_t in_stride,
                                                              __nv_bfloat16* __restrict__ out, int64_t out_stride, int rows,
                                                              int inter, int gelu) {
  const int c = blockIdx.x * kActThreads + threadIdx.x;
  if (c * 8 >= inter) return;
  for (int t = blockIdx.y * 2; t < rows; t += gridDim.y * 2) {
    const __nv_bfloat16* r0 = gate_up + t * in_stride + c * 8;
    const bool two = t + 1 < rows;
    const uint4 g0 = *reinterpret_cast<const uint4*>(r0);
    const uint4 u0 = *reinterpret_cast<const uint4*>(r0 + inter);
    uint4 g1 = g0, u1 = u0;
    if (two) {
      g1 = *reinterpret_cast<const uint4*>(r0 + in_stride);
      u1 = *reinterpret_cast<const uint4*>(r0 + in_stride + inter);
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + c * 8) = act_mul8(g0, u0, gelu);
    if (two) *reinterpret_cast<uint4*>(out + (t + 1) * out_stride + c * 8) = act_mul8(g1, u1, gelu);
  }
}

// One CTA per row.  y' = y (or rmsnorm(y, y_weight) rounded to bf16);  x = bf16(x + y');
// out = rmsnorm(x, weight).  Norms are fp32: v * rsqrt(mean(v^2) + eps) * w  (or * (1 + w)).
constexpr int kNormThreads = 256;                            // the most threads a row gets

template <int NT>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();                                           // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) s += scratch[w];
  return s;
}

// VPT 8-element vectors per thread, NT threads per row (hidden <= NT * 8 * VPT).  Rows of up to 1024 elements take
// 128 threads: twice the rows per SM, so twice the loads in flight.  Both operands of a row are requested
// before anything is reduced.
template <int VPT, int NT>
__global__ void __launch_bounds__(NT) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ y, int64_t y_stride,
                                                                  const __nv_bfloat16* __restrict__ y_weight,
                                                                  const __nv_bfloat16* __restrict__ weight,
                                                                  __nv_bfloat16* __restrict__ out, int hidden,
                                                                  float eps, int unit_offset,
                                                                  const int32_t* __restrict__ row_ends) {
  __shared__ float scratch[NT / 32];
  // row_ends != nullptr: output row r is computed from source row row_ends[r + 1] - 1 (the last token of
  // sequence r of a packed prefill batch) and the residual stream is left as it is
  const int out_row = blockIdx.x;
  const int row = row_ends != nullptr ? row_ends[out_row + 1] - 1 : out_row;
  if (row < 0) return;                                       // (an empty batch prefix: nothing to read)
  const int nvec = hidden / 8;
  const float one = unit_offset ? 1.f : 0.f;
  float xv[VPT][8];
  uint4 res[VPT];                                            // the residual stream's vectors, requested up front
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * NT;
    res[k] = make_uint4(0, 0, 0, 0);
    if (v < nvec) res[k] = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * hidden + v * 8);
  }
  // ---- branch output, optionally normalised first (Gemma's post-attention / post-feedforward norm)
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * NT;
    if (v < nvec) {
      const uint4 yv = *reinterpret_cast<const uint4*>(y + row * y_stride + v * 8);
      const uint32_t* ya = reinterpret_cast<const uint32_t*>(&yv);
#pragma unroll
      for (int i = 0; i < 4; ++i) { xv[k][2 * i] = bf16_lo(ya[i]); xv[k][2 * i + 1] = bf16_hi(ya[i]); }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += xv[k][i] * xv[k][i];
    }
  }
  if (y_weight != nullptr) {
    const float rstd = rsqrtf(block_sum<NT>(ss, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * NT;
      if (v < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(y_weight + v * 8);
        const uint32_t* wa = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          xv[k][2 * i] = round_bf16(xv[k][2 * i] * rstd * (one + bf16_lo(wa[i])));
          xv[k][2 * i + 1] = round_bf16(xv[k][2 * i + 1] * rstd * (one + bf16_hi(wa[i])));
        }
      }
    }
  }
  // ---- residual add (rounded to bf16, written back) and the norm of the new residual stream
  ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * NT;
    if (v < nvec) {
      uint4 rv = res[k];
      uint32_t* ra = reinterpret_cast<uint32_t*>(&rv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ra[i] = pack_bf16(bf16_lo(ra[i]) + xv[k][2 * i], bf16_hi(ra[i]) + xv[k][2 * i + 1]);
        xv[k][2 * i] = bf16_lo(ra[i]); xv[k][2 * i + 1] = bf16_hi(ra[i]);
      }
      if (row_ends == nullptr) *reinterpret_cast<uint4*>(x + static_cast<int64_t>(row) * hidden + v * 8) = rv;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += xv[k][i] * xv[k][i];
    }
  }
  const float rstd = rsqrtf(block_sum<NT>(ss, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * NT;
    if (v < nvec) {
      const uint4 wv = *reinterpret_cast<const uint4*>(weight + v * 8);
      const uint32_t* wa = reinterpret_cast<const uint32_t*>(&wv);
      uint4 ov;
      uint32_t* oa = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        oa[i] = pack_bf16(xv[k][2 * i] * rstd * (one + bf16_lo(wa[i])), xv[k][2 * i + 1] * rstd * (one + bf16_hi(wa[i])));
      *reinterpret_cast<uint4*>(out + static_cast<int64_t>(out_row) * hidden + v * 8) = ov;
    }
  }
}

static bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mvb

extern "C" int mvb_act_mul(const void* gate_up, int64_t in_row_stride, void* out, int64_t out_row_stride, int rows,
                           int intermediate, int gelu_tanh, void* stream) {
  using namespace mvb;
  if (!gate_up || !out || rows < 0 || intermediate <= 0) return kInvalidArgument;
  if (intermediate % 8 || in_row_stride % 8 || out_row_stride % 8 || !a16(gate_up) || !a16(out)) return kMisaligned;
  if (rows == 0) return kOk;
  const int bx = (intermediate / 8 + kActThreads - 1) / kActThreads;
  int by = (rows + 1) / 2;                                     // row pairs
  const int cap = (sm_count() * 16 + bx - 1) / bx;             // about 16 blocks of 128 threads per SM
  if (by > cap) by = cap;
  if (by > 65535) by = 65535;
  act_mul_kernel<<<dim3(bx, by), kActThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), in_row_stride, static_cast<__nv_bfloat16*>(out), out_row_stride, rows,
      intermediate, gelu_tanh);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

static int add_rmsnorm_impl(void* x, const void* y, int64_t y_row_stride, const void* y_weight, const void* weight,
                            void* out, const int32_t* row_ends, int rows, int hidden, float eps, int unit_offset,
                            void* stream) {
  using namespace mvb;
  if (!x || !y || !weight || !out || rows < 0 || hidden <= 0) return kInvalidArgument;
  if (hidden % 8 || y_row_stride % 8 || !a16(x) || !a16(y) || !a16(weight) || !a16(out) || !a16(y_weight)) return kMisaligned;
  if (hidden > kNormThreads * 8 * 4) return kUnsupportedShape;
  if (rows == 0) return kOk;
  auto* xp = static_cast<__nv_bfloat16*>(x);
  auto* yp = static_cast<const __nv_bfloat16*>(y);
  auto* ywp = static_cast<const __nv_bfloat16*>(y_weight);
  auto* wp = static_cast<const __nv_bfloat16*>(weight);
  auto* op = static_cast<__nv_bfloat16*>(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vpt = (hidden / 8 + kNormThreads - 1) / kNormThreads;
  if (hidden <= 128 * 8) add_rmsnorm_kernel<1, 128><<<rows, 128, 0, st>>>(xp, yp, y_row_stride, ywp, wp, op, hidden, eps, unit_offset, row_ends);
  else if (vpt <= 1) add_rmsnorm_kernel<1, kNormThreads><<<rows, kNormThreads, 0, st>>>(xp, yp, y_row_stride, ywp, wp, op, hidden, eps, unit_offset, row_ends);
  else if (vpt == 2) add_rmsnorm_kernel<2, kNormThreads><<<rows, kNormThreads, 0, st>>>(xp, yp, y_row_stride, ywp, wp, op, hidden, eps, unit_offset, row_ends);
  else add_rmsnorm_kernel<4, kNormThreads><<<rows, kNormThreads, 0, st>>>(xp, yp, y_row_stride, ywp, wp, op, hidden, eps, unit_offset, row_ends);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

extern "C" int mvb_add_rmsnorm(void* x, const void* y, int64_t y_row_stride, const void* y_weight, const void* weight,
                               void* out, int rows, int hidden, float eps, int unit_offset, void* stream) {
  return add_rmsnorm_impl(x, y, y_row_stride, y_weight, weight, out, nullptr, rows, hidden, eps, unit_offset, stream);
}

extern "C" int mvb_add_rmsnorm_last_tokens(const void* x, const void* y, int64_t y_row_stride, const void* y_weight,
                                           const void* weight, void* out, const int32_t* cu_seqlens_q, int num_seqs,
                                           int hidden, float eps, int unit_offset, void* stream) {
  if (!cu_seqlens_q) return mvb::kInvalidArgument;
  return add_rmsnorm_impl(const_cast<void*>(x), y, y_row_stride, y_weight, weight, out, cu_seqlens_q, num_seqs, hidden,
                          eps, unit_offset, stream);
}
