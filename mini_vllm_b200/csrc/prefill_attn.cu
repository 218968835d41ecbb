// Causal varlen prefill attention over dense or paged K/V on the tcgen05 tensor cores.
//
// One CTA (128 threads) owns a 128-row query tile of one (sequence, query head) and walks the
// visible KV tiles of BN tokens:
//   TMA (128-byte swizzle) stages Q once and K/V tiles through two-deep rings; K/V tiles of the
//   paged pool are addressed through the block table (a tile never straddles a block);
//   S = Q K^T      tcgen05.mma, M=128, N=BN, fp32 accumulator in tensor memory (two S buffers,
//                  so the next tile's QK^T runs under this tile's softmax);
//   softmax        thread r owns row r: tcgen05.ld brings its row of S into registers, so the
//                  running max / sum need no shuffles; P is written to shared memory as bf16 in
//                  the K-major swizzled layout the tensor core reads;
//   O += P V       tcgen05.mma with V consumed MN-major straight from the TMA layout; O stays
//                  in tensor memory and is rescaled there only when the running max moved by
//                  more than 2^8 (the stale max is carried exactly through P and the row sum).
// Epilogue: O / l -> bf16 -> global, 256 bytes per row.
//
// Roofline: tensor-bound, 4 * D flops per (query, key) pair per head.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

namespace mvb {

struct PrefillParams {
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* block_table;   // nullptr: dense K/V
  int64_t table_stride;
  int block_size;
  int64_t kv_rows;
  int num_seqs, hq, group;
  float scale_log2;
  int window_left;
  __nv_bfloat16* out;
  int64_t out_stride;
  int* dev_status;
};

template <int D, int BN>
struct PrefillCfg {
  static constexpr int BM = 128;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;          // one K (or V) tile
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int HALF_Q = BM * 128;              // bytes of one 64-column half of Q / P
  static constexpr int HALF_KV = BN * 128;             // bytes of one 64-column half of K / V
  static constexpr int SMEM = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 512;
  static constexpr int S0_COL = 0, S1_COL = BN, O_COL = 2 * BN;
  static_assert(2 * BN + D <= 512, "tensor memory budget");
};

template <int D, int BN>
__global__ void __launch_bounds__(128, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
  using C = PrefillCfg<D, BN>;
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, BN, false, false);
  constexpr uint32_t IDESC_O = umma_idesc_bf16(128, D, false, true);
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5;
  const int s = blockIdx.y, qh = blockIdx.z;
  const int kvh = qh / p.group;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int k0 = p.cu_k[s], k_len = p.cu_k[s + 1] - k0;
  // longest tiles first: the last query tile of a causal sequence has the most keys
  const int n_qt = (q_len + 127) / 128;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  if (qt < 0) return;                                         // CTA-uniform
  const int row0 = qt * 128;
  const int rows = min(128, q_len - row0);
  const int shift = k_len - q_len;                            // position of query row 0
  const int p_first = shift + row0, p_last = shift + row0 + rows - 1;
  const int j_lo = p.window_left >= 0 ? max(0, p_first - p.window_left) / BN : 0;
  const int j_hi = p_last / BN;
  const int n_it = j_hi - j_lo + 1;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base;
  const uint32_t k_s = q_s + C::Q_BYTES;                      // 2 stages
  const uint32_t v_s = k_s + 2 * C::KV_BYTES;                 // 2 stages
  const uint32_t p_s = v_s + 2 * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + C::Q_BYTES + 4 * C::KV_BYTES + C::P_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* v_full = bars + 3;        // [2]
  uint64_t* s_done = bars + 5;        // [2]
  uint64_t* o_done = bars + 7;        // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  uint32_t* fail_flag = tmem_slot + 1;

  if (tid == 0) {
    tma_prefetch_desc(&q_map); tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map);
    for (int i = 0; i < 8; ++i) mbar_init(&bars[i], 1);
    *fail_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  // first KV row (tensor-map z coordinate) of tile j of this sequence
  auto kv_row = [&](int j) -> int {
    const int tok = j * BN;
    if (p.block_table == nullptr) return k0 + tok;
    const int blk = p.block_table[s * p.table_stride + tok / p.block_size];
    if (blk < 0 || static_cast<int64_t>(blk + 1) * p.block_size > p.kv_rows) {
      report(p.dev_status, kDevBadBlock, s);
      return -BN;                                             // fully out of range: zero fill
    }
    return blk * p.block_size + tok % p.block_size;
  };
  auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint64_t* bar, int j) {
    const int z = kv_row(j);
    mbar_arrive_expect_tx(bar, C::KV_BYTES);
#pragma unroll
    for (int h = 0; h < D / 64; ++h) {
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
          ::"r"(dst + h * C::HALF_KV), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(h * 64),
            "r"(kvh), "r"(z) : "memory");
    }
  };
  auto issue_s = [&](int it) {                                // S[it&1] = Q . K_it^T
    const uint32_t kb = k_s + (it & 1) * C::KV_BYTES;
    const uint32_t d = tmem + ((it & 1) ? C::S1_COL : C::S0_COL);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint64_t a = umma_desc_sw128(q_s + (ks >> 2) * C::HALF_Q + (ks & 3) * 32, 16, 1024);
      const uint64_t b = umma_desc_sw128(kb + (ks >> 2) * C::HALF_KV + (ks & 3) * 32, 16, 1024);
      umma_bf16_ss(d, a, b, IDESC_S, ks > 0);
    }
    umma_commit(&s_done[it & 1]);
  };
  // A failed wait poisons the CTA: everybody skips the rest but still reaches the barriers.
  auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int where) {
    if (!mbar_wait(bar, parity)) {
      report(p.dev_status, kDevWaitTimeout, where);
      atomicExch(fail_flag, 1u);
    }
  };

  if (tid == 0) {
    mbar_arrive_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
    for (int h = 0; h < D / 64; ++h) {
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
          ::"r"(q_s + h * C::HALF_Q), "l"(reinterpret_cast<uint64_t>(&q_map)), "r"(smem_u32(q_full)), "r"(h * 64),
            "r"(qh), "r"(q0 + row0) : "memory");
    }
    for (int it = 0; it < 2 && it < n_it; ++it) {
      load_tile(&k_map, k_s + it * C::KV_BYTES, &k_full[it], j_lo + it);
      load_tile(&v_map, v_s + it * C::KV_BYTES, &v_full[it], j_lo + it);
    }
    wait_or_fail(q_full, 0, 100);
    wait_or_fail(&k_full[0], 0, 101);
    tc_fence_after();
    issue_s(0);
  }

  const int my_pos = p_first + tid;                           // absolute position of this thread's row
  float m_run = -INFINITY, l_run = 0.f;
  bool failed = false;

  for (int it = 0; it < n_it && !failed; ++it) {
    const int st = it & 1;
    const int j = j_lo + it;
    wait_or_fail(&s_done[st], (it >> 1) & 1, 200 + it);
    tc_fence_after();
    if (tid == 0) {
      if (it + 2 < n_it) load_tile(&k_map, k_s + st * C::KV_BYTES, &k_full[st], j + 2);   // K stage st is free
      if (it + 1 < n_it) {
        wait_or_fail(&k_full[st ^ 1], ((it + 1) >> 1) & 1, 300 + it);
        tc_fence_after();
        issue_s(it + 1);
      }
    }

    // ---- softmax on row tid of S[st] -------------------------------------------------------------
    const uint32_t s_addr = lane_addr + (st ? C::S1_COL : C::S0_COL);
    const int col0 = j * BN;
    const bool need_mask = (col0 + BN - 1 > p_first) || (p.window_left >= 0 && col0 < p_last - p.window_left);
    const int hi_key = my_pos;                                              // last visible key
    const int lo_key = p.window_left >= 0 ? my_pos - p.window_left : 0;     // first visible key
    float tile_max = -INFINITY;
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(s_addr + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float x = __uint_as_float(r[i]);
        if (need_mask) {
          const int key = col0 + c * 32 + i;
          if (key > hi_key || key < lo_key) x = -INFINITY;
        }
        tile_max = fmaxf(tile_max, x);
      }
    }
    tile_max *= p.scale_log2;                                 // scale > 0, so max commutes with it
    // lazy rescale: keep the old max unless the new one is more than 2^8 larger
    float m_use = m_run, alpha = 1.f;
    if (tile_max > m_run + 8.f || (m_run == -INFINITY && tile_max > -INFINITY)) {
      m_use = tile_max;
      alpha = fast_exp2(m_run - m_use);                       // m_run = -inf -> 0
    }
    const bool warp_rescale = __any_sync(0xffffffffu, alpha != 1.f) && it > 0;
    const float m_safe = m_use == -INFINITY ? 0.f : m_use;

    if (it > 0) {                                             // P, O and V stage st^1 are busy until PV(it-1) is done
      wait_or_fail(o_done, (it - 1) & 1, 400 + it);
      tc_fence_after();
      if (tid == 0 && it + 1 < n_it) load_tile(&v_map, v_s + (st ^ 1) * C::KV_BYTES, &v_full[st ^ 1], j + 1);
    }

    float row_sum = 0.f;
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(s_addr + c * 32, r);
      tmem_wait_ld();
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float x0 = __uint_as_float(r[i]), x1 = __uint_as_float(r[i + 1]);
        if (need_mask) {
          const int key = col0 + c * 32 + i;
          if (key > hi_key || key < lo_key) x0 = -INFINITY;
          if (key + 1 > hi_key || key + 1 < lo_key) x1 = -INFINITY;
        }
        const float e0 = fast_exp2(fmaf(x0, p.scale_log2, -m_safe));
        const float e1 = fast_exp2(fmaf(x1, p.scale_log2, -m_safe));
        row_sum += e0 + e1;
        packed[i >> 1] = pack_bf16(e0, e1);
      }
      // 32 columns = 4 chunks of 16 bytes of row tid, K-major 128-byte swizzle
      const uint32_t half = (c * 32) / 64, chunk0 = ((c * 32) % 64) / 8;
      const uint32_t rb = p_s + half * C::HALF_Q + tid * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rb + (((chunk0 + q) ^ (tid & 7)) << 4)),
                     "r"(packed[4 * q]), "r"(packed[4 * q + 1]), "r"(packed[4 * q + 2]), "r"(packed[4 * q + 3])
                     : "memory");
      }
    }
    l_run = l_run * alpha + row_sum;
    m_run = m_use;

    if (warp_rescale) {                                       // warp-uniform: tcgen05.ld/st are warp-collective
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + C::O_COL + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_32x32(lane_addr + C::O_COL + c * 32, r);
      }
      tmem_wait_st();
    }

    // V tile: rows past the end of the sequence may hold anything; zero them before the MMA reads
    wait_or_fail(&v_full[st], (it >> 1) & 1, 500 + it);
    {
      const int valid = k_len - col0;
      if (valid < BN && tid >= valid && tid < BN) {
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
#pragma unroll
          for (int q = 0; q < 8; ++q)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_s + st * C::KV_BYTES + h * C::HALF_KV + tid * 128 + q * 16),
                         "r"(0) : "memory");
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    failed = *reinterpret_cast<volatile uint32_t*>(fail_flag) != 0;
    if (tid == 0 && !failed) {
      tc_fence_after();
      const uint32_t vb = v_s + st * C::KV_BYTES;
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
        const uint64_t a = umma_desc_sw128(p_s + (ks >> 2) * C::HALF_Q + (ks & 3) * 32, 16, 1024);
        const uint64_t b = umma_desc_sw128(vb + ks * 2048, C::HALF_KV, 1024);
        umma_bf16_ss(tmem + C::O_COL, a, b, IDESC_O, (it > 0 || ks > 0) ? 1u : 0u);
      }
      umma_commit(o_done);
    }
  }

  // ---- epilogue -----------------------------------------------------------------------------------
  if (!failed) {
    wait_or_fail(o_done, (n_it - 1) & 1, 600);
    tc_fence_after();
    failed = *reinterpret_cast<volatile uint32_t*>(fail_flag) != 0;
  }
  if (!failed) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.out + (static_cast<int64_t>(q0) + row0 + tid) * p.out_stride + static_cast<int64_t>(qh) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(lane_addr + C::O_COL + c * 32, r);
      tmem_wait_ld();
      if (tid < rows) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(r[8 * q + 0]) * inv, __uint_as_float(r[8 * q + 1]) * inv);
          w.y = pack_bf16(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv);
          w.z = pack_bf16(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv);
          w.w = pack_bf16(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = w;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <int D, int BN>
static int launch_prefill(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const PrefillParams& p,
                          int max_seqlen_q, cudaStream_t stream) {
  using C = PrefillCfg<D, BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attn_kernel<D, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
      return kLaunchFailed;
    configured = true;
  }
  dim3 grid((max_seqlen_q + 127) / 128, p.num_seqs, p.hq);
  prefill_attn_kernel<D, BN><<<grid, 128, C::SMEM, stream>>>(qm, km, vm, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace mvb

extern "C" int mvb_prefill_attn(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                const void* v, int64_t v_row_stride, int64_t kv_rows, const int32_t* cu_seqlens_q,
                                const int32_t* cu_seqlens_k, const int32_t* block_table, int64_t table_stride,
                                int block_size, int num_seqs, int total_q, int max_seqlen_q, int num_q_heads,
                                int num_kv_heads, int head_dim, float scale, int window_left, void* out,
                                int64_t out_row_stride, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (!q || !k || !v || !cu_seqlens_q || !cu_seqlens_k || !out) return kInvalidArgument;
  if (num_seqs <= 0 || total_q < 0 || max_seqlen_q < 0 || kv_rows <= 0) return kInvalidArgument;
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return kInvalidArgument;
  if (head_dim != 128 && head_dim != 256) return kUnsupportedShape;
  const int bn = head_dim == 128 ? 128 : 64;
  if (block_table != nullptr && (block_size <= 0 || block_size % bn != 0)) return kUnsupportedShape;
  if (kv_rows > 0x7fffffffLL || num_seqs > 65535 || num_q_heads > 65535) return kUnsupportedShape;
  if (total_q == 0 || max_seqlen_q == 0) return kOk;
  if ((out_row_stride % 8) != 0 || !is_aligned(out, 16)) return kMisaligned;

  CUtensorMap qm, km, vm;
  int rc = make_kv_tensor_map(&qm, q, total_q, num_q_heads, head_dim, q_row_stride, 128);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&km, k, kv_rows, num_kv_heads, head_dim, k_row_stride, bn);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&vm, v, kv_rows, num_kv_heads, head_dim, v_row_stride, bn);
  if (rc != kOk) return rc;

  PrefillParams p;
  p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k; p.block_table = block_table; p.table_stride = table_stride;
  p.block_size = block_size; p.kv_rows = kv_rows; p.num_seqs = num_seqs; p.hq = num_q_heads;
  p.group = num_q_heads / num_kv_heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window_left = window_left;
  p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_row_stride;
  p.dev_status = dev_status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_prefill<128, 128>(qm, km, vm, p, max_seqlen_q, st);
  return launch_prefill<256, 64>(qm, km, vm, p, max_seqlen_q, st);
}
