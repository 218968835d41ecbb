// Causal varlen prefill attention over dense or paged K/V on the tcgen05 tensor cores.
//
// One CTA owns NQ query tiles of 128 rows of one (sequence, query head) and walks the visible KV
// tiles of BN tokens.  Warps are specialised:
//   producer warp   TMA (128-byte swizzle, no multicast): the Q tiles once, then K and V tiles
//                   through two-deep rings; KV tiles of the paged pool are addressed through the
//                   block table (a tile never straddles a block); zero-fills V rows past the end
//                   of the sequence (pool slots that were never written may hold NaNs);
//   MMA warp        one thread issues every tcgen05.mma: S_t = Q_t K^T (M=128, N=BN, fp32
//                   accumulators in tensor memory) and O_t += P_t V with P read from tensor
//                   memory (it overwrites S in place as packed bf16) and V consumed MN-major
//                   straight from the TMA layout.  The two query tiles are interleaved
//                   (S0, PV1, S1, PV0, ...) so the tensor pipe works on one tile while the other
//                   tile's softmax runs;
//   softmax groups  one warpgroup per query tile, one thread per row: tcgen05.ld brings the row of
//                   S into registers (no shuffles), running max / sum, exp2, P back to tensor
//                   memory, O rescaled in tensor memory only when the running max moved by more
//                   than 2^8 (the stale max is carried exactly through P and the row sum), and the
//                   epilogue O / l -> bf16 -> global.
// Every mbarrier wait is bounded; a wait that gives up poisons the CTA, which then drains.
//
// Roofline: tensor-bound, 4 * D flops per (query, key) pair per head.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

#include <type_traits>

namespace mvb {

// Optional phase timers (only with -DMVB_PREFILL_TRACE): one CTA accumulates SM-clock deltas per
// phase in registers and writes them once at the end.
#ifdef MVB_PREFILL_TRACE
__device__ unsigned long long* g_prefill_trace = nullptr;
#define MVB_PT_DECL long long pt_acc_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long pt_last_ = clock64();
#define MVB_PTRACE(role, it, code)                                   \
  do {                                                               \
    const long long now_ = clock64();                                \
    pt_acc_[(code)] += now_ - pt_last_;                              \
    pt_last_ = now_;                                                 \
  } while (0)
#define MVB_PT_FLUSH(role)                                                                        \
  do {                                                                                            \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && g_prefill_trace)                 \
      for (int i_ = 0; i_ < 8; ++i_) g_prefill_trace[(role) * 8 + i_] = pt_acc_[i_];              \
  } while (0)
#else
#define MVB_PT_DECL
#define MVB_PTRACE(role, it, code)
#define MVB_PT_FLUSH(role)
#endif

struct PrefillParams {
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* block_table;   // nullptr: dense K/V
  int64_t table_stride;
  int block_size;
  int64_t kv_rows;
  int num_seqs, hq, group;
  int pair_heads;               // 1: the CTA's query tiles are the heads of one GQA group over the same rows
  float scale_log2;
  int window_left;
  __nv_bfloat16* out;
  int64_t out_stride;
  int* dev_status;
};

template <int D, int BN, int NQ>
struct PrefillCfg {
  static constexpr int THREADS = NQ * 128 + 64;
  static constexpr int Q_BYTES = 128 * D * 2;          // one query tile
  static constexpr int KV_BYTES = BN * D * 2;          // one K (or V) tile
  static constexpr int HALF_Q = 128 * 128;             // bytes of one 64-column half of a Q tile
  static constexpr int HALF_KV = BN * 128;             // bytes of one 64-column half of K / V
  static constexpr int SMEM = NQ * Q_BYTES + 4 * KV_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = NQ * (BN + D) <= 256 ? 256 : 512;   // power of two; <= 256 lets two CTAs share an SM
  static constexpr int S_COL = 0;                      // S_t at S_COL + t * BN (P_t aliases its first BN/2 columns)
  static constexpr int O_COL = NQ * BN;                // O_t at O_COL + t * D
  static_assert(NQ * (BN + D) <= 512, "tensor memory budget");
  static_assert(BN % 64 == 0, "P is written in 64-key halves");
};

// barrier slots
// P is published in 64-key halves (slot B_PFULL + 2 * tile + half) so the PV product of the first
// half starts while the second half is still being exponentiated.
enum : int { B_QFULL = 0, B_KFULL = 2, B_VFULL = 4, B_KFREE = 6, B_VFREE = 8, B_SFULL = 10, B_PFULL = 12,
             B_ODONE = 16, B_VFIXED = 18, B_COUNT = 19 };

template <int D, int BN, int NQ>
__global__ void __launch_bounds__(PrefillCfg<D, BN, NQ>::THREADS, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
  using C = PrefillCfg<D, BN, NQ>;
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, BN, false, false);
  constexpr uint32_t IDESC_O = umma_idesc_bf16(128, D, false, true);
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The NQ query tiles of a CTA are either NQ heads of one GQA group over the same 128 rows (each
  // K/V tile loaded once serves them all: half the K/V traffic per flop) or, without a group to share,
  // NQ consecutive 128-row tiles of one head.
  const bool pair = p.pair_heads != 0;
  // grid = (heads or head pairs, sequences, query-block rank): blocks are dispatched x-fastest, so every
  // sequence's LAST query block (the one with the most keys) is handed out before any second-to-last one,
  // which keeps the tail of the launch short
  const int s = blockIdx.y, qh0 = pair ? blockIdx.x * NQ : blockIdx.x;
  const int kvh = qh0 / p.group;
  const int rows_per_cta = pair ? 128 : 128 * NQ;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int k0 = p.cu_k[s], k_len = p.cu_k[s + 1] - k0;
  // longest blocks first: the last query block of a causal sequence has the most keys
  const int n_qb = (q_len + rows_per_cta - 1) / rows_per_cta;
  const int qb = n_qb - 1 - static_cast<int>(blockIdx.z);
  if (qb < 0) return;                                         // CTA-uniform
  const int row0 = qb * rows_per_cta;
  const int shift = k_len - q_len;                            // position of query row 0

  // per query tile: rows, first/last position, KV tile range
  int rows_t[NQ], pf_t[NQ], pl_t[NQ], jlo_t[NQ], jhi_t[NQ], roff_t[NQ], head_t[NQ];
  int j_lo = 0x7fffffff, j_hi = -1;
#pragma unroll
  for (int t = 0; t < NQ; ++t) {
    roff_t[t] = pair ? 0 : 128 * t;
    head_t[t] = pair ? qh0 + t : qh0;
    rows_t[t] = max(0, min(128, q_len - row0 - roff_t[t]));
    pf_t[t] = shift + row0 + roff_t[t];
    pl_t[t] = pf_t[t] + rows_t[t] - 1;
    jlo_t[t] = p.window_left >= 0 ? max(0, pf_t[t] - p.window_left) / BN : 0;
    jhi_t[t] = rows_t[t] > 0 ? pl_t[t] / BN : -1;
    if (rows_t[t] > 0) { j_lo = min(j_lo, jlo_t[t]); j_hi = max(j_hi, jhi_t[t]); }
  }
  const int n_it = j_hi - j_lo + 1;
  auto active = [&](int t, int j) { return rows_t[t] > 0 && j >= jlo_t[t] && j <= jhi_t[t]; };

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base;                                  // NQ tiles
  const uint32_t k_s = q_s + NQ * C::Q_BYTES;                 // 2 stages
  const uint32_t v_s = k_s + 2 * C::KV_BYTES;                 // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + NQ * C::Q_BYTES + 4 * C::KV_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile uint32_t* fail_flag = tmem_slot + 1;

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(&bars[i], (i >= B_PFULL && i < B_PFULL + 4) ? 128u : 1u);
    *fail_flag = 0;
    fence_mbar_init();
  }
  if (warp == NQ * 4 + 1) {                                   // the MMA warp owns the tensor memory
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Bounded wait that also gives up when another role has failed.
  auto wait = [&](int slot, uint32_t parity, int where) -> bool {
    for (int spin = 0; spin < 64; ++spin) {
      if (mbar_wait(&bars[slot], parity, 1u << 14)) return true;
      if (*fail_flag) return false;
    }
    report(p.dev_status, kDevWaitTimeout, where);
    *fail_flag = 1;
    return false;
  };

  if (warp == NQ * 4) {
    // ============================ producer warp ======================================================
    auto kv_row = [&](int j) -> int {                         // tensor-map row of KV tile j of this sequence
      const int tok = j * BN;
      if (p.block_table == nullptr) return k0 + tok;
      const int blk = p.block_table[s * p.table_stride + tok / p.block_size];
      if (blk < 0 || static_cast<int64_t>(blk + 1) * p.block_size > p.kv_rows) {
        report(p.dev_status, kDevBadBlock, s);
        return -BN;                                           // fully out of range: zero fill
      }
      return blk * p.block_size + tok % p.block_size;
    };
    auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint64_t* bar, int z) {
      mbar_arrive_expect_tx(bar, C::KV_BYTES);
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst + h * C::HALF_KV), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(h * 64),
              "r"(kvh), "r"(z) : "memory");
      }
    };
    if (lane == 0) {
      tma_prefetch_desc(&q_map); tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map);
#pragma unroll
      for (int t = 0; t < NQ; ++t) {
        if (rows_t[t] <= 0) continue;
        mbar_arrive_expect_tx(&bars[B_QFULL + t], C::Q_BYTES);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(q_s + t * C::Q_BYTES + h * C::HALF_Q), "l"(reinterpret_cast<uint64_t>(&q_map)),
                "r"(smem_u32(&bars[B_QFULL + t])), "r"(h * 64), "r"(head_t[t]), "r"(q0 + row0 + roff_t[t]) : "memory");
        }
      }
    }
    bool ok = true;
    MVB_PT_DECL
    for (int it = 0; it < n_it && ok; ++it) {
      const int st = it & 1, j = j_lo + it;
      if (lane == 0) {
        const int z = kv_row(j);
        if (it >= 2) ok = wait(B_KFREE + st, ((it >> 1) - 1) & 1, 100 + it);
        if (ok) load_tile(&k_map, k_s + st * C::KV_BYTES, &bars[B_KFULL + st], z);
        MVB_PTRACE(0, it, 0);
        if (ok && it >= 2) ok = wait(B_VFREE + st, ((it >> 1) - 1) & 1, 200 + it);
        if (ok) load_tile(&v_map, v_s + st * C::KV_BYTES, &bars[B_VFULL + st], z);
        MVB_PTRACE(0, it, 1);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const int valid = k_len - j * BN;
      if (ok && valid < BN) {                                 // last, partial tile: zero V rows past the end
        ok = wait(B_VFULL + st, (it >> 1) & 1, 300 + it);
        if (ok) {
          for (int r = max(valid, 0) + lane; r < BN; r += 32) {
#pragma unroll
            for (int h = 0; h < D / 64; ++h)
#pragma unroll
              for (int q = 0; q < 8; ++q)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_s + st * C::KV_BYTES + h * C::HALF_KV + r * 128 + q * 16),
                             "r"(0) : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[B_VFIXED]);
        }
      }
    }
    if (lane == 0) { MVB_PT_FLUSH(0); }
  } else if (warp == NQ * 4 + 1) {
    // ============================ MMA warp (one issuing thread) ======================================
    // This thread shares its scheduler with two softmax warps that always have work, so every
    // instruction between two tcgen05.mma costs tensor-pipe time: ranges are scalars, tile indices
    // are compile-time constants and a wait is one try_wait unless the barrier is really not ready.
    if (lane == 0) {
      bool ok = true;
      MVB_PT_DECL
      const uint64_t q_desc0 = umma_desc_sw128(q_s, 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(k_s, 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(v_s, C::HALF_KV, 1024);
      const int jlo0 = jlo_t[0], jhi0 = jhi_t[0];
      const int jlo1 = jlo_t[NQ - 1], jhi1 = jhi_t[NQ - 1];   // tile NQ-1 (== tile 0 when NQ == 1)
      const int j_partial = k_len / BN;                       // first KV tile with rows past the end
      auto ready = [&](int slot, uint32_t parity, int where) -> bool {
        return mbar_try_wait(&bars[slot], parity) ? true : wait(slot, parity, where);
      };
      auto issue_s = [&](auto tt, int st) {                   // S_t = Q_t . K^T
        constexpr int t = decltype(tt)::value;
        const uint64_t qd = q_desc0 + ((t * C::Q_BYTES) >> 4), kd = k_desc0 + ((st * C::KV_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t qo = ((ks >> 2) * C::HALF_Q + (ks & 3) * 32) >> 4, ko = ((ks >> 2) * C::HALF_KV + (ks & 3) * 32) >> 4;
          umma_bf16_ss(tmem + C::S_COL + t * BN, qd + qo, kd + ko, IDESC_S, ks > 0);
        }
        umma_commit(&bars[B_SFULL + t]);
      };
      // O_t (+)= P_t . V for KV tile j: V must have landed (and been fixed up if partial); the halves
      // of P_t are consumed as the softmax group publishes them
      auto pv_step = [&](auto tt, int it, bool v_known) {
        constexpr int t = decltype(tt)::value;
        const int st = it & 1, j = j_lo + it;
        const int jlo = t == 0 ? jlo0 : jlo1;
        if (!v_known) {
          ok = ready(B_VFULL + st, (it >> 1) & 1, 400 + it);
          if (ok && j >= j_partial) ok = ready(B_VFIXED, 0, 450);
        }
        MVB_PTRACE(1, it, 6);
        const uint64_t vd = v_desc0 + ((st * C::KV_BYTES) >> 4);
        const uint32_t first = (j == jlo) ? 0u : 1u;
#pragma unroll
        for (int h = 0; h < BN / 64; ++h) {
          if (ok) ok = ready(B_PFULL + 2 * t + h, (j - jlo) & 1, 500 + it);
          if (!ok) return;
          tc_fence_after();
          MVB_PTRACE(1, it, 7);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int ks = h * 4 + k4;
            umma_bf16_ts(tmem + C::O_COL + t * D, tmem + C::S_COL + t * BN + ks * 8, vd + ((ks * 2048) >> 4), IDESC_O,
                         ks > 0 ? 1u : first);
          }
          MVB_PTRACE(1, it, (t == 0 ? 5 : 3));
        }
        umma_commit(&bars[B_ODONE + t]);
      };
      using T0 = std::integral_constant<int, 0>;
      using T1 = std::integral_constant<int, NQ - 1>;
      bool prev_a0 = false, prev_a1 = false;                  // was tile 0 / tile NQ-1 active in the previous step
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1, j = j_lo + it;
        MVB_PTRACE(1, it, 0);
        ok = ready(B_KFULL + st, (it >> 1) & 1, 600 + it);
        if (!ok) break;
        tc_fence_after();
        MVB_PTRACE(1, it, 1);
        const bool a0 = j >= jlo0 && j <= jhi0;
        // interleave the tiles: S0(j), PV1(j-1), S1(j), PV0(j)
        if (a0) {
          if (j == jlo0) ok = ready(B_QFULL + 0, 0, 610);
          if (ok) issue_s(T0{}, st);
        }
        MVB_PTRACE(1, it, 2);
        if constexpr (NQ > 1) {
          if (it >= 1 && ok) {
            if (prev_a1) pv_step(T1{}, it - 1, prev_a0);      // tile 0's PV already waited for that V tile
            if (ok) umma_commit(&bars[B_VFREE + ((it - 1) & 1)]);
          }
          MVB_PTRACE(1, it, 3);
          const bool a1 = rows_t[NQ - 1] > 0 && j >= jlo1 && j <= jhi1;
          if (ok && a1) {
            if (j == jlo1) ok = ready(B_QFULL + NQ - 1, 0, 611);
            if (ok) issue_s(T1{}, st);
          }
          prev_a1 = a1;
        }
        if (ok) umma_commit(&bars[B_KFREE + st]);
        MVB_PTRACE(1, it, 4);
        if (ok && a0) pv_step(T0{}, it, false);
        MVB_PTRACE(1, it, 5);
        if (NQ == 1 && ok) umma_commit(&bars[B_VFREE + st]);
        prev_a0 = a0;
      }
      if constexpr (NQ > 1) {
        if (ok) {
          if (prev_a1) pv_step(T1{}, n_it - 1, prev_a0);
          if (ok) umma_commit(&bars[B_VFREE + ((n_it - 1) & 1)]);
        }
      }
      MVB_PT_FLUSH(1);
    }
    __syncwarp();
  } else {
    // ============================ softmax warpgroup of query tile t ==================================
    const int t = warp >> 2;
    const int row = tid & 127;                                // row of the tile = TMEM lane
    if (rows_t[t] > 0) {
      const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
      const uint32_t s_addr = lane_addr + C::S_COL + t * BN;
      const uint32_t o_addr = lane_addr + C::O_COL + t * D;
      const int my_pos = pf_t[t] + row;                       // absolute position of this row's query
      const int hi_key = my_pos;
      const int lo_key = p.window_left >= 0 ? my_pos - p.window_left : 0;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      MVB_PT_DECL
      const int n_itt = jhi_t[t] - jlo_t[t] + 1;
      for (int itt = 0; itt < n_itt && ok; ++itt) {
        const int j = jlo_t[t] + itt, col0 = j * BN;
        if (row == 0) MVB_PTRACE(2 + t, itt, 0);
        ok = wait(B_SFULL + t, itt & 1, 700 + itt);
        if (!ok) break;
        tc_fence_after();
        if (row == 0) MVB_PTRACE(2 + t, itt, 1);
        const bool need_mask = (col0 + BN - 1 > pf_t[t]) || (p.window_left >= 0 && col0 < pl_t[t] - p.window_left);
        // visible keys of this row inside the tile: [vis_lo, vis_hi] relative to col0 (only used when masking)
        const int vis_lo = lo_key - col0, vis_hi = hi_key - col0;
        // pass 1: row maximum (two code paths so the common unmasked tile carries no mask arithmetic)
        float tile_max = -INFINITY;
#pragma unroll
        for (int hf = 0; hf < BN / 64; ++hf) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(s_addr + hf * 64, r0);
          tmem_ld_32x32(s_addr + hf * 64 + 32, r1);
          tmem_wait_ld();
          if (!need_mask) {
            float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              m0 = fmaxf(m0, __uint_as_float(r0[i]));
              m1 = fmaxf(m1, __uint_as_float(r1[i]));
            }
            tile_max = fmaxf(tile_max, fmaxf(m0, m1));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int c0 = hf * 64 + i, c1 = c0 + 32;
              const float x0 = (c0 >= vis_lo && c0 <= vis_hi) ? __uint_as_float(r0[i]) : -INFINITY;
              const float x1 = (c1 >= vis_lo && c1 <= vis_hi) ? __uint_as_float(r1[i]) : -INFINITY;
              tile_max = fmaxf(tile_max, fmaxf(x0, x1));
            }
          }
        }
        if (row == 0) MVB_PTRACE(2 + t, itt, 2);
        tile_max *= p.scale_log2;                             // scale > 0, so max commutes with it
        // lazy rescale: keep the old max unless the new one is more than 2^8 larger
        float m_use = m_run, alpha = 1.f;
        if (tile_max > m_run + 8.f || (m_run == -INFINITY && tile_max > -INFINITY)) {
          m_use = tile_max;
          alpha = fast_exp2(m_run - m_use);                   // m_run = -inf -> 0
        }
        const float m_safe = m_use == -INFINITY ? 0.f : m_use;
        // S_t(itt) complete implies PV_t(itt-1) complete (one thread issues both, in order), so O is ours
        if (itt > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(o_addr + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, r);
          }
        }
        if (row == 0) MVB_PTRACE(2 + t, itt, 3);
        // pass 2: P = exp2(S * scale - m) as packed bf16 over the first BN/2 columns of S, published per half
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int hf = 0; hf < BN / 64; ++hf) {
          uint32_t r0[32], r1[32], pk[32];
          tmem_ld_32x32(s_addr + hf * 64, r0);
          tmem_ld_32x32(s_addr + hf * 64 + 32, r1);
          tmem_wait_ld();
          if (!need_mask) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(r0[i]), p.scale_log2, -m_safe));
              const float e1 = fast_exp2(fmaf(__uint_as_float(r0[i + 1]), p.scale_log2, -m_safe));
              const float f0 = fast_exp2(fmaf(__uint_as_float(r1[i]), p.scale_log2, -m_safe));
              const float f1 = fast_exp2(fmaf(__uint_as_float(r1[i + 1]), p.scale_log2, -m_safe));
              sum0 += e0 + e1; sum1 += f0 + f1;
              pk[i >> 1] = pack_bf16(e0, e1);                 // keys hf*64 + i, i+1      -> word (hf*64 + i)/2
              pk[16 + (i >> 1)] = pack_bf16(f0, f1);          // keys hf*64 + 32 + i, ... -> word 16 + ...
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int c0 = hf * 64 + i, c1 = c0 + 32;
              const float a0 = (c0 >= vis_lo && c0 <= vis_hi) ? __uint_as_float(r0[i]) : -INFINITY;
              const float a1 = (c0 + 1 >= vis_lo && c0 + 1 <= vis_hi) ? __uint_as_float(r0[i + 1]) : -INFINITY;
              const float b0 = (c1 >= vis_lo && c1 <= vis_hi) ? __uint_as_float(r1[i]) : -INFINITY;
              const float b1 = (c1 + 1 >= vis_lo && c1 + 1 <= vis_hi) ? __uint_as_float(r1[i + 1]) : -INFINITY;
              const float e0 = fast_exp2(fmaf(a0, p.scale_log2, -m_safe)), e1 = fast_exp2(fmaf(a1, p.scale_log2, -m_safe));
              const float f0 = fast_exp2(fmaf(b0, p.scale_log2, -m_safe)), f1 = fast_exp2(fmaf(b1, p.scale_log2, -m_safe));
              sum0 += e0 + e1; sum1 += f0 + f1;
              pk[i >> 1] = pack_bf16(e0, e1);
              pk[16 + (i >> 1)] = pack_bf16(f0, f1);
            }
          }
          tmem_st_32x32(s_addr + hf * 32, pk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&bars[B_PFULL + 2 * t + hf]);
        }
        l_run = l_run * alpha + (sum0 + sum1);
        m_run = m_use;
        if (row == 0) MVB_PTRACE(2 + t, itt, 4);
      }
      if (row == 0) { MVB_PT_FLUSH(2 + t); }
      // ---- epilogue ---------------------------------------------------------------------------------
      if (ok) ok = wait(B_ODONE + t, (n_itt - 1) & 1, 800);
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow = p.out + (static_cast<int64_t>(q0) + row0 + roff_t[t] + row) * p.out_stride +
                              static_cast<int64_t>(head_t[t]) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c * 32, r);
          tmem_wait_ld();
          if (row < rows_t[t]) {
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
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == NQ * 4 + 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

struct PrefillOperands {            // what the tensor maps are built from
  const void *q, *k, *v;
  int64_t q_stride, k_stride, v_stride, kv_rows;
  int total_q, hq, hkv;
};

template <int D, int BN, int NQ>
static int launch_prefill(const PrefillOperands& op, const PrefillParams& p, int max_seqlen_q, cudaStream_t stream) {
  using C = PrefillCfg<D, BN, NQ>;
  if (p.block_table != nullptr && p.block_size % BN != 0) return kUnsupportedShape;   // a KV tile must not straddle blocks
  // the TMA boxes are tied to the kernel's tile sizes: 128 query rows, BN key rows
  CUtensorMap qm, km, vm;
  int rc = make_kv_tensor_map(&qm, op.q, op.total_q, op.hq, D, op.q_stride, 128);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&km, op.k, op.kv_rows, op.hkv, D, op.k_stride, BN);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&vm, op.v, op.kv_rows, op.hkv, D, op.v_stride, BN);
  if (rc != kOk) return rc;
  static bool configured_by_device[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured_by_device[dev & 63]) {
    if (cudaFuncSetAttribute(prefill_attn_kernel<D, BN, NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) !=
        cudaSuccess)
      return kLaunchFailed;
    configured_by_device[dev & 63] = true;
  }
  PrefillParams pp = p;
  pp.pair_heads = (NQ > 1 && p.group % NQ == 0) ? 1 : 0;
  const int rows_per_cta = pp.pair_heads ? 128 : 128 * NQ;
  dim3 grid(pp.pair_heads ? p.hq / NQ : p.hq, p.num_seqs, (max_seqlen_q + rows_per_cta - 1) / rows_per_cta);
  if (grid.z > 65535) return kUnsupportedShape;
  prefill_attn_kernel<D, BN, NQ><<<grid, C::THREADS, C::SMEM, stream>>>(qm, km, vm, pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace mvb

#ifdef MVB_PREFILL_TRACE
extern "C" int mvb_debug_set_prefill_trace(void* ptr) {
  unsigned long long* p = static_cast<unsigned long long*>(ptr);
  return cudaMemcpyToSymbol(mvb::g_prefill_trace, &p, sizeof(p)) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" int mvb_prefill_attn(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                const void* v, int64_t v_row_stride, int64_t kv_rows,
                                const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* block_table, int64_t table_stride, int block_size, int num_seqs,
                                int total_q, int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                                float scale, int window_left, void* out, int64_t out_row_stride,
                                int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (!q || !k || !v || !cu_seqlens_q || !cu_seqlens_k || !out) return kInvalidArgument;
  if (num_seqs <= 0 || total_q < 0 || max_seqlen_q < 0 || kv_rows <= 0) return kInvalidArgument;
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return kInvalidArgument;
  if (head_dim != 128 && head_dim != 256) return kUnsupportedShape;
  if (block_table != nullptr && block_size <= 0) return kInvalidArgument;
  if (kv_rows > 0x7fffffffLL || num_seqs > 65535 || num_q_heads > 65535) return kUnsupportedShape;
  if (total_q == 0 || max_seqlen_q == 0) return kOk;
  if ((out_row_stride % 8) != 0 || !is_aligned(out, 16)) return kMisaligned;

  const PrefillOperands op{q, k, v, q_row_stride, k_row_stride, v_row_stride, kv_rows, total_q, num_q_heads, num_kv_heads};

  PrefillParams p;
  p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k; p.block_table = block_table; p.table_stride = table_stride;
  p.block_size = block_size; p.kv_rows = kv_rows; p.num_seqs = num_seqs; p.hq = num_q_heads;
  p.group = num_q_heads / num_kv_heads;
  p.pair_heads = 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window_left = window_left;
  p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_row_stride;
  p.dev_status = dev_status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_prefill<128, 128, 2>(op, p, max_seqlen_q, st);
  return launch_prefill<256, 64, 1>(op, p, max_seqlen_q, st);
}
