// Fused rotary embedding + paged KV-cache write (HBM-bound elementwise pass).
//
// One thread owns one 16-byte chunk pair: 8 bf16 of the first half of a head and the matching
// 8 of the second half (rotate-half pairs element i with i + D/2), or one 16-byte chunk of V.
// q is rotated in place, k is rotated and scattered to the cache slot (and optionally written
// back), v is copied to the cache slot.  All global accesses are 128-bit.
//
// Algorithmic bytes per token: (Hq + 2*Hkv) * D * 2 read + (Hq + 2*Hkv) * D * 2 written
// (+ the token's cos/sin row, 4*D bytes, shared by all heads through L1/L2).
#include "common.cuh"
#include "mini_vllm_b200.h"

namespace mvb {

struct RopeParams {
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t q_stride, k_stride, v_stride;
  const int64_t* positions;
  const float* cos_sin;
  int64_t max_pos;
  const int32_t* slot_mapping;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int64_t num_slots;
  int num_tokens, hq, hkv, d;
  int k_in_place;
  int* dev_status;
};

// Rounds exactly like the eager fp32 reference: each product and the sum are rounded on
// their own (no FMA contraction), then one round-to-nearest-even to bf16.
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float* cs, const float* sn) {
  uint32_t* a = reinterpret_cast<uint32_t*>(&lo);
  uint32_t* b = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float x1a = bf16_lo(a[i]), x1b = bf16_hi(a[i]);
    float x2a = bf16_lo(b[i]), x2b = bf16_hi(b[i]);
    float c0 = cs[2 * i], c1 = cs[2 * i + 1], s0 = sn[2 * i], s1 = sn[2 * i + 1];
    float y1a = __fsub_rn(__fmul_rn(x1a, c0), __fmul_rn(x2a, s0));
    float y1b = __fsub_rn(__fmul_rn(x1b, c1), __fmul_rn(x2b, s1));
    float y2a = __fadd_rn(__fmul_rn(x2a, c0), __fmul_rn(x1a, s0));
    float y2b = __fadd_rn(__fmul_rn(x2b, c1), __fmul_rn(x1b, s1));
    a[i] = pack_bf16(y1a, y1b);
    b[i] = pack_bf16(y2a, y2b);
  }
}

__global__ void __launch_bounds__(256) rope_kv_write_kernel(const RopeParams p) {
  const int pairs_per_head = p.d / 16;                       // chunk pairs per head
  const int rope_tasks = (p.hq + p.hkv) * pairs_per_head;    // per token
  const int v_tasks = p.hkv * p.d / 8;
  const int tasks = rope_tasks + v_tasks;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<int64_t>(p.num_tokens) * tasks) return;
  const int t = static_cast<int>(gid / tasks);
  const int task = static_cast<int>(gid - static_cast<int64_t>(t) * tasks);

  int64_t slot = -1;
  if (p.slot_mapping != nullptr) {
    slot = p.slot_mapping[t];
    if (slot >= p.num_slots || slot < -1) {
      report(p.dev_status, kDevBadSlot, t);
      slot = -1;
    }
  }

  if (task >= rope_tasks) {                                  // ---- V: plain copy to the cache slot
    if (slot < 0) return;
    const int c = task - rope_tasks;                         // 16-byte chunk within the token's V row
    const uint4 val = *reinterpret_cast<const uint4*>(p.v + t * p.v_stride + c * 8);
    *reinterpret_cast<uint4*>(p.v_cache + slot * (static_cast<int64_t>(p.hkv) * p.d) + c * 8) = val;
    return;
  }

  const int head = task / pairs_per_head;                    // 0..hq-1 are q heads, then k heads
  const int c = task - head * pairs_per_head;                // chunk pair within the head
  const bool is_q = head < p.hq;
  __nv_bfloat16* row = is_q ? p.q + t * p.q_stride + head * p.d : p.k + t * p.k_stride + (head - p.hq) * p.d;
  if (!is_q && slot < 0 && !p.k_in_place) return;            // nothing to produce for this k chunk
  if (is_q && p.cos_sin == nullptr) return;                  // plain store_kvcache leaves q alone

  uint4 lo = *reinterpret_cast<const uint4*>(row + c * 8);
  uint4 hi = *reinterpret_cast<const uint4*>(row + p.d / 2 + c * 8);
  if (p.cos_sin != nullptr) {
    const int64_t pos = p.positions[t];
    if (pos < 0 || pos >= p.max_pos) {
      report(p.dev_status, kDevBadPosition, t);
    } else {
      const float* tab = p.cos_sin + pos * p.d;
      float cs[8], sn[8];
      *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(tab + c * 8);
      *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(tab + c * 8 + 4);
      *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(tab + p.d / 2 + c * 8);
      *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(tab + p.d / 2 + c * 8 + 4);
      rotate8(lo, hi, cs, sn);
    }
  }
  if (is_q || p.k_in_place) {
    if (p.cos_sin != nullptr) {
      *reinterpret_cast<uint4*>(row + c * 8) = lo;
      *reinterpret_cast<uint4*>(row + p.d / 2 + c * 8) = hi;
    }
  }
  if (!is_q && slot >= 0) {
    __nv_bfloat16* dst = p.k_cache + slot * (static_cast<int64_t>(p.hkv) * p.d) + (head - p.hq) * p.d;
    *reinterpret_cast<uint4*>(dst + c * 8) = lo;
    *reinterpret_cast<uint4*>(dst + p.d / 2 + c * 8) = hi;
  }
}

// ---- variant with the per-head RMSNorm of q and k fused in front of the rotation ------------------
// q/k/v are read where the projection GEMM left them (row strides of the packed output), each head
// row is normalised in fp32 (y = x * rsqrt(mean(x^2) + eps) * w, or * (1 + w) for Gemma), rounded to
// bf16 as the separate norm kernel would, rotated, and written: q in place, k to the cache (and in
// place when asked), v to the cache.  The D/16 threads of a head row are consecutive lanes, so the
// sum of squares is a shuffle reduction inside an aligned lane group.
struct NormRopeParams {
  RopeParams r;
  const __nv_bfloat16* q_weight;
  const __nv_bfloat16* k_weight;
  float eps;
  int unit_offset;
};

__global__ void __launch_bounds__(256) qk_norm_rope_kv_write_kernel(const NormRopeParams np) {
  const RopeParams& p = np.r;
  const int pairs_per_head = p.d / 16;
  const int rope_tasks = (p.hq + p.hkv) * pairs_per_head;
  const int v_tasks = p.hkv * p.d / 8;
  const int tasks = rope_tasks + v_tasks;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool in_range = gid < static_cast<int64_t>(p.num_tokens) * tasks;
  const int t = in_range ? static_cast<int>(gid / tasks) : 0;
  const int task = in_range ? static_cast<int>(gid - static_cast<int64_t>(t) * tasks) : tasks;   // tasks = idle
  const bool is_rope = task < rope_tasks;

  int64_t slot = -1;
  if (in_range && p.slot_mapping != nullptr) {
    slot = p.slot_mapping[t];
    if (slot >= p.num_slots || slot < -1) {
      report(p.dev_status, kDevBadSlot, t);
      slot = -1;
    }
  }
  if (in_range && !is_rope && slot >= 0) {                   // V: plain copy to the cache slot
    const int c = task - rope_tasks;
    const uint4 val = *reinterpret_cast<const uint4*>(p.v + t * p.v_stride + c * 8);
    *reinterpret_cast<uint4*>(p.v_cache + slot * (static_cast<int64_t>(p.hkv) * p.d) + c * 8) = val;
  }

  const int head = is_rope ? task / pairs_per_head : 0;
  const int c = is_rope ? task - head * pairs_per_head : 0;
  const bool is_q = head < p.hq;
  __nv_bfloat16* row = is_q ? p.q + t * p.q_stride + head * p.d : p.k + t * p.k_stride + (head - p.hq) * p.d;
  uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
  float ss = 0.f;
  if (is_rope) {
    lo = *reinterpret_cast<const uint4*>(row + c * 8);
    hi = *reinterpret_cast<const uint4*>(row + p.d / 2 + c * 8);
    const uint32_t* a = reinterpret_cast<const uint32_t*>(&lo);
    const uint32_t* b = reinterpret_cast<const uint32_t*>(&hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x0 = bf16_lo(a[i]), x1 = bf16_hi(a[i]), y0 = bf16_lo(b[i]), y1 = bf16_hi(b[i]);
      ss += x0 * x0 + x1 * x1 + y0 * y0 + y1 * y1;
    }
  }
  // every thread of the warp takes part; a head's lanes form an aligned group of pairs_per_head
  for (int off = 1; off < pairs_per_head; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (!is_rope) return;
  if (!is_q && slot < 0 && !p.k_in_place) return;

  const float rstd = rsqrtf(ss / static_cast<float>(p.d) + np.eps);
  const __nv_bfloat16* w = is_q ? np.q_weight : np.k_weight;
  {
    const uint4 wl = *reinterpret_cast<const uint4*>(w + c * 8);
    const uint4 wh = *reinterpret_cast<const uint4*>(w + p.d / 2 + c * 8);
    uint32_t* a = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* b = reinterpret_cast<uint32_t*>(&hi);
    const uint32_t* wa = reinterpret_cast<const uint32_t*>(&wl);
    const uint32_t* wb = reinterpret_cast<const uint32_t*>(&wh);
    const float one = np.unit_offset ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[i] = pack_bf16(bf16_lo(a[i]) * rstd * (one + bf16_lo(wa[i])), bf16_hi(a[i]) * rstd * (one + bf16_hi(wa[i])));
      b[i] = pack_bf16(bf16_lo(b[i]) * rstd * (one + bf16_lo(wb[i])), bf16_hi(b[i]) * rstd * (one + bf16_hi(wb[i])));
    }
  }
  const int64_t pos = p.positions[t];
  if (pos < 0 || pos >= p.max_pos) {
    report(p.dev_status, kDevBadPosition, t);
  } else {
    const float* tab = p.cos_sin + pos * p.d;
    float cs[8], sn[8];
    *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(tab + c * 8);
    *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(tab + c * 8 + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(tab + p.d / 2 + c * 8);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(tab + p.d / 2 + c * 8 + 4);
    rotate8(lo, hi, cs, sn);
  }
  if (is_q || p.k_in_place) {
    *reinterpret_cast<uint4*>(row + c * 8) = lo;
    *reinterpret_cast<uint4*>(row + p.d / 2 + c * 8) = hi;
  }
  if (!is_q && slot >= 0) {
    __nv_bfloat16* dst = p.k_cache + slot * (static_cast<int64_t>(p.hkv) * p.d) + (head - p.hq) * p.d;
    *reinterpret_cast<uint4*>(dst + c * 8) = lo;
    *reinterpret_cast<uint4*>(dst + p.d / 2 + c * 8) = hi;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mvb

extern "C" int mvb_rope_kv_write(void* q, int64_t q_row_stride, void* k, int64_t k_row_stride, const void* v,
                                 int64_t v_row_stride, const int64_t* positions, const float* cos_sin,
                                 int64_t max_pos, const int32_t* slot_mapping, void* k_cache, void* v_cache,
                                 int64_t num_slots, int num_tokens, int num_q_heads, int num_kv_heads,
                                 int head_dim, int k_in_place, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (num_tokens < 0 || num_q_heads < 0 || num_kv_heads <= 0 || head_dim <= 0) return kInvalidArgument;
  if (head_dim % 16 != 0) return kUnsupportedShape;
  if (num_tokens == 0) return kOk;
  if (k == nullptr || v == nullptr || (num_q_heads > 0 && q == nullptr)) return kInvalidArgument;
  if (cos_sin != nullptr && positions == nullptr) return kInvalidArgument;
  if (slot_mapping != nullptr && (k_cache == nullptr || v_cache == nullptr || num_slots <= 0)) return kInvalidArgument;
  if ((q_row_stride % 8) || (k_row_stride % 8) || (v_row_stride % 8)) return kMisaligned;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(k_cache) || !aligned16(v_cache) ||
      !aligned16(cos_sin))
    return kMisaligned;
  RopeParams p;
  p.q = static_cast<__nv_bfloat16*>(q);
  p.k = static_cast<__nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_stride = q_row_stride; p.k_stride = k_row_stride; p.v_stride = v_row_stride;
  p.positions = positions; p.cos_sin = cos_sin; p.max_pos = max_pos;
  p.slot_mapping = slot_mapping;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.num_slots = num_slots;
  p.num_tokens = num_tokens; p.hq = num_q_heads; p.hkv = num_kv_heads; p.d = head_dim;
  p.k_in_place = k_in_place;
  p.dev_status = dev_status;
  const int64_t tasks = static_cast<int64_t>(num_q_heads + num_kv_heads) * (head_dim / 16) +
                        static_cast<int64_t>(num_kv_heads) * head_dim / 8;
  const int64_t total = tasks * num_tokens;
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return kInvalidArgument;
  rope_kv_write_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

extern "C" int mvb_qk_norm_rope_kv_write(void* q, int64_t q_row_stride, void* k, int64_t k_row_stride, const void* v,
                                         int64_t v_row_stride, const void* q_weight, const void* k_weight, float eps,
                                         int unit_offset, const int64_t* positions, const float* cos_sin,
                                         int64_t max_pos, const int32_t* slot_mapping, void* k_cache, void* v_cache,
                                         int64_t num_slots, int num_tokens, int num_q_heads, int num_kv_heads,
                                         int head_dim, int k_in_place, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (num_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return kInvalidArgument;
  const int pph = head_dim / 16;
  if (head_dim % 16 != 0 || pph > 32 || (pph & (pph - 1)) != 0) return kUnsupportedShape;   // lane groups
  if (num_tokens == 0) return kOk;
  if (!q || !k || !v || !q_weight || !k_weight || !positions || !cos_sin) return kInvalidArgument;
  if (slot_mapping != nullptr && (k_cache == nullptr || v_cache == nullptr || num_slots <= 0)) return kInvalidArgument;
  if ((q_row_stride % 8) || (k_row_stride % 8) || (v_row_stride % 8)) return kMisaligned;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(k_cache) || !aligned16(v_cache) ||
      !aligned16(cos_sin) || !aligned16(q_weight) || !aligned16(k_weight))
    return kMisaligned;
  NormRopeParams np;
  RopeParams& p = np.r;
  p.q = static_cast<__nv_bfloat16*>(q);
  p.k = static_cast<__nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_stride = q_row_stride; p.k_stride = k_row_stride; p.v_stride = v_row_stride;
  p.positions = positions; p.cos_sin = cos_sin; p.max_pos = max_pos;
  p.slot_mapping = slot_mapping;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.num_slots = num_slots;
  p.num_tokens = num_tokens; p.hq = num_q_heads; p.hkv = num_kv_heads; p.d = head_dim;
  p.k_in_place = k_in_place;
  p.dev_status = dev_status;
  np.q_weight = static_cast<const __nv_bfloat16*>(q_weight);
  np.k_weight = static_cast<const __nv_bfloat16*>(k_weight);
  np.eps = eps; np.unit_offset = unit_offset;
  const int64_t tasks = static_cast<int64_t>(num_q_heads + num_kv_heads) * pph + static_cast<int64_t>(num_kv_heads) * head_dim / 8;
  if (tasks % pph != 0) return kUnsupportedShape;
  const int64_t blocks = (tasks * num_tokens + 255) / 256;
  if (blocks > 0x7fffffffLL) return kInvalidArgument;
  qk_norm_rope_kv_write_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(np);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}
