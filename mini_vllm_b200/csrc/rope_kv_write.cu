// Fused rotary embedding + paged KV-cache write (HBM-bound elementwise pass), optionally with the per-head
// RMSNorm of q and k in front.
//
// q is rotated in place, k is rotated and scattered to the cache slot (and optionally written back), v is
// copied to the cache slot.  All global accesses are 128-bit; rotate-half pairs element i with i + D/2, so a
// task is one 16-byte chunk of the first half of a head together with its partner in the second half.
//
// Algorithmic bytes per token: (Hq + 2*Hkv) * D * 2 read + (Hq + 2*Hkv) * D * 2 written
// (+ the token's cos/sin row, 4*D bytes, shared by all heads through L1/L2).
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

#include <type_traits>

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

// EXACT rounds exactly like the eager fp32 reference: each product and the sum are rounded on their own (no FMA
// contraction), then one round-to-nearest-even to bf16.  Without it one product of each pair is fused into
// the sum (a third fewer instructions): the result can differ in the last fp32 bit, i.e. almost never after
// the rounding to bf16; used where bit-exactness is not promised (the variant with the norm fused in front).
template <bool EXACT>
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float* cs, const float* sn) {
  uint32_t* a = reinterpret_cast<uint32_t*>(&lo);
  uint32_t* b = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float x1a = bf16_lo(a[i]), x1b = bf16_hi(a[i]);
    float x2a = bf16_lo(b[i]), x2b = bf16_hi(b[i]);
    float c0 = cs[2 * i], c1 = cs[2 * i + 1], s0 = sn[2 * i], s1 = sn[2 * i + 1];
    float y1a, y1b, y2a, y2b;
    if (EXACT) {
      y1a = __fsub_rn(__fmul_rn(x1a, c0), __fmul_rn(x2a, s0));
      y1b = __fsub_rn(__fmul_rn(x1b, c1), __fmul_rn(x2b, s1));
      y2a = __fadd_rn(__fmul_rn(x2a, c0), __fmul_rn(x1a, s0));
      y2b = __fadd_rn(__fmul_rn(x2b, c1), __fmul_rn(x1b, s1));
    } else {
      y1a = fmaf(x1a, c0, -__fmul_rn(x2a, s0));
      y1b = fmaf(x1b, c1, -__fmul_rn(x2b, s1));
      y2a = fmaf(x2a, c0, __fmul_rn(x1a, s0));
      y2b = fmaf(x2b, c1, __fmul_rn(x1b, s1));
    }
    a[i] = pack_bf16(y1a, y1b);
    b[i] = pack_bf16(y2a, y2b);
  }
}

// ---- the kernel ------------------------------------------------------------------------------------------
// A token's work is (Hq + Hkv) * D/16 rotation tasks (a 16-byte chunk of the first half of a head with its
// partner in the second half) followed by Hkv * D/8 copy tasks (a 16-byte chunk of V).  A warp takes ITEMS
// consecutive groups of 32 tasks of ONE token: every lane first issues all its loads (up to 2 * ITEMS
// independent 128-bit loads, plus the token's slot, position and cos/sin entries), then rotates and stores.
// With D/16 dividing 32 a lane meets the same chunk index in every group, so its cos/sin values are loaded
// once per token.  ITEMS is chosen on the host: large for long prefills (bytes in flight per thread bound the
// bandwidth), 1 for decode batches (enough warps to cover the GPU matter more).  Three blocks per SM: with
// five groups per warp the kernel is otherwise held to two by its registers, and measured a fifth slower.
//
// NORM adds the per-head RMSNorm of q and k in front of the rotation: each head row is normalised in fp32
// (y = x * rsqrt(mean(x^2) + eps) * w, or * (1 + w) for Gemma), rounded to bf16 as the separate norm kernel
// would, then rotated.  The D/16 lanes of a head row are consecutive lanes of an aligned group, so the sum of
// squares is a shuffle reduction inside the group.
struct NormRopeParams {
  RopeParams r;
  const __nv_bfloat16* q_weight;
  const __nv_bfloat16* k_weight;
  float eps;
  int unit_offset;
};

// PPH fixes the chunk pairs per head at compile time (8: head_dim 128, 16: head_dim 256; 0: read it from the
// parameters), which turns the task -> (head, chunk) divisions of every group into shifts.
template <int ITEMS, bool NORM, int PPH>
__global__ void __launch_bounds__(256, 3) rope_kv_kernel(const NormRopeParams np) {
  const RopeParams& p = np.r;
  const int pph = PPH ? PPH : p.d / 16;                      // chunk pairs per head
  const int d = PPH ? PPH * 16 : p.d;
  const int rope_tasks = (p.hq + p.hkv) * pph;               // per token
  const int tasks = rope_tasks + p.hkv * d / 8;
  const int groups = (tasks + 31) >> 5;
  const int warps_per_token = (groups + ITEMS - 1) / ITEMS;
  const int lane = threadIdx.x & 31;
  int64_t t64;
  int warp_in_token;
  if (gridDim.x <= 0x0fffffffu) {                            // the usual case: a 32-bit division
    const uint32_t gwarp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t q = gwarp / static_cast<uint32_t>(warps_per_token);
    t64 = q;
    warp_in_token = static_cast<int>(gwarp - q * static_cast<uint32_t>(warps_per_token));
  } else {
    const int64_t gwarp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    t64 = gwarp / warps_per_token;
    warp_in_token = static_cast<int>(gwarp - t64 * warps_per_token);
  }
  if (t64 >= p.num_tokens) return;                           // warp-uniform
  const int t = static_cast<int>(t64);
  const int task0 = warp_in_token * (ITEMS * 32) + lane;
  const bool rotate = p.cos_sin != nullptr;

  // ---- every load of this lane goes out before anything is used ------------------------------------------
  int64_t slot = p.slot_mapping != nullptr ? static_cast<int64_t>(p.slot_mapping[t]) : -1;
  const int64_t pos = rotate ? p.positions[t] : 0;
  uint4 lo[ITEMS], hi[ITEMS];
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const int task = task0 + 32 * j;
    lo[j] = make_uint4(0, 0, 0, 0); hi[j] = make_uint4(0, 0, 0, 0);
    if (task < rope_tasks) {
      const int head = task / pph, c = task - head * pph;
      const __nv_bfloat16* row = head < p.hq ? p.q + t * p.q_stride + head * d : p.k + t * p.k_stride + (head - p.hq) * d;
      lo[j] = *reinterpret_cast<const uint4*>(row + c * 8);
      hi[j] = *reinterpret_cast<const uint4*>(row + d / 2 + c * 8);
    } else if (task < tasks) {
      lo[j] = *reinterpret_cast<const uint4*>(p.v + t * p.v_stride + (task - rope_tasks) * 8);
    }
  }
  if (slot >= p.num_slots || slot < -1) {
    report(p.dev_status, kDevBadSlot, t);
    slot = -1;
  }
  const bool pos_ok = pos >= 0 && pos < p.max_pos;
  if (rotate && !pos_ok && task0 < rope_tasks) report(p.dev_status, kDevBadPosition, t);
  const bool same_chunk = (32 % pph) == 0;                   // the lane's chunk index does not depend on the group
  float cs[8], sn[8];
  auto load_table = [&](int c) {
    const float* tab = p.cos_sin + pos * d;
    *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(tab + c * 8);
    *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(tab + c * 8 + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(tab + d / 2 + c * 8);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(tab + d / 2 + c * 8 + 4);
  };
  if (rotate && pos_ok && same_chunk && task0 < rope_tasks) load_table(task0 % pph);

  // ---- rotate and store -------------------------------------------------------------------------------------
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const int task = task0 + 32 * j;
    const bool is_rope = task < rope_tasks;
    const int head = is_rope ? task / pph : 0;
    const int c = is_rope ? task - head * pph : 0;
    const bool is_q = head < p.hq;
    if (NORM) {
      float ss = 0.f;
      if (is_rope) {
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&lo[j]);
        const uint32_t* b = reinterpret_cast<const uint32_t*>(&hi[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = bf16_lo(a[i]), x1 = bf16_hi(a[i]), y0 = bf16_lo(b[i]), y1 = bf16_hi(b[i]);
          ss += x0 * x0 + x1 * x1 + y0 * y0 + y1 * y1;
        }
      }
      // every lane of the warp takes part; a head's lanes form an aligned group of pph
      for (int off = 1; off < pph; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (is_rope && (is_q || slot >= 0 || p.k_in_place)) {
        const float rstd = rsqrtf(ss / static_cast<float>(d) + np.eps);
        const __nv_bfloat16* w = is_q ? np.q_weight : np.k_weight;
        const uint4 wl = *reinterpret_cast<const uint4*>(w + c * 8);
        const uint4 wh = *reinterpret_cast<const uint4*>(w + d / 2 + c * 8);
        uint32_t* a = reinterpret_cast<uint32_t*>(&lo[j]);
        uint32_t* b = reinterpret_cast<uint32_t*>(&hi[j]);
        const uint32_t* wa = reinterpret_cast<const uint32_t*>(&wl);
        const uint32_t* wb = reinterpret_cast<const uint32_t*>(&wh);
        const float one = np.unit_offset ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          a[i] = pack_bf16(bf16_lo(a[i]) * rstd * (one + bf16_lo(wa[i])), bf16_hi(a[i]) * rstd * (one + bf16_hi(wa[i])));
          b[i] = pack_bf16(bf16_lo(b[i]) * rstd * (one + bf16_lo(wb[i])), bf16_hi(b[i]) * rstd * (one + bf16_hi(wb[i])));
        }
      }
    }
    if (task >= tasks) continue;
    if (!is_rope) {                                          // ---- V: plain copy to the cache slot
      if (slot >= 0)
        *reinterpret_cast<uint4*>(p.v_cache + slot * (static_cast<int64_t>(p.hkv) * d) + (task - rope_tasks) * 8) = lo[j];
      continue;
    }
    if (!is_q && slot < 0 && !p.k_in_place) continue;        // nothing to produce for this k chunk
    if (is_q && !rotate && !NORM) continue;                  // plain store_kvcache leaves q alone
    if (rotate && pos_ok) {
      if (!same_chunk) load_table(c);
      rotate8<!NORM>(lo[j], hi[j], cs, sn);
    }
    __nv_bfloat16* row = is_q ? p.q + t * p.q_stride + head * d : p.k + t * p.k_stride + (head - p.hq) * d;
    if ((is_q || p.k_in_place) && (rotate || NORM)) {
      *reinterpret_cast<uint4*>(row + c * 8) = lo[j];
      *reinterpret_cast<uint4*>(row + d / 2 + c * 8) = hi[j];
    }
    if (!is_q && slot >= 0) {
      __nv_bfloat16* dst = p.k_cache + slot * (static_cast<int64_t>(p.hkv) * d) + (head - p.hq) * d;
      *reinterpret_cast<uint4*>(dst + c * 8) = lo[j];
      *reinterpret_cast<uint4*>(dst + d / 2 + c * 8) = hi[j];
    }
  }
}

template <bool NORM>
static int launch_rope(const NormRopeParams& np, cudaStream_t stream) {
  const RopeParams& p = np.r;
  const int64_t tasks = static_cast<int64_t>(p.hq + p.hkv) * (p.d / 16) + static_cast<int64_t>(p.hkv) * p.d / 8;
  const int64_t groups = (tasks + 31) / 32;
  // enough warps to give every SM a few blocks come first; beyond that, more loads in flight per thread
  const int64_t want_warps = static_cast<int64_t>(sm_count()) * 32;
  int items = 1;
  if (groups >= 5 && p.num_tokens * ((groups + 4) / 5) >= want_warps) items = 5;
  else if (groups >= 2 && p.num_tokens * ((groups + 1) / 2) >= want_warps) items = 2;
  const int64_t warps = p.num_tokens * ((groups + items - 1) / items);
  const int64_t blocks = (warps * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return kInvalidArgument;
  const unsigned grid = static_cast<unsigned>(blocks);
  auto launch = [&](auto pph_tag) {
    constexpr int PPH = decltype(pph_tag)::value;
    if (items == 5) rope_kv_kernel<5, NORM, PPH><<<grid, 256, 0, stream>>>(np);
    else if (items == 2) rope_kv_kernel<2, NORM, PPH><<<grid, 256, 0, stream>>>(np);
    else rope_kv_kernel<1, NORM, PPH><<<grid, 256, 0, stream>>>(np);
  };
  if (p.d == 128) launch(std::integral_constant<int, 8>{});
  else if (p.d == 256) launch(std::integral_constant<int, 16>{});
  else launch(std::integral_constant<int, 0>{});
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
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
  NormRopeParams np;
  np.r = p;
  np.q_weight = np.k_weight = nullptr; np.eps = 0.f; np.unit_offset = 0;
  return launch_rope<false>(np, static_cast<cudaStream_t>(stream));
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
  return launch_rope<true>(np, static_cast<cudaStream_t>(stream));
}
