// Causal varlen prefill attention over dense or paged K/V on the tcgen05 tensor cores.
//
// A work item is NQ query tiles of 128 rows of one (sequence, query head or head pair); it walks the
// visible KV tiles of BN tokens.  The grid has one block index per item, but a CTA does not end with
// its item: through cluster launch control it takes over the index of a CTA that has not started yet
// and carries on with its barriers, tensor memory and K/V rings alive, so the loads and first products
// of the next item overlap the epilogue of the current one and nothing is set up twice.
// Warps are specialised:
//   producer warp   fetches items (skipping block indices past a sequence's last query block) and
//                   publishes them to the other roles; TMA (128-byte swizzle, no multicast): the Q
//                   tiles of an item, then K and V tiles through two-deep rings; KV tiles of the
//                   paged pool are addressed through the block table (a tile never straddles a
//                   block); zero-fills V rows past the end of the sequence (pool slots that were
//                   never written may hold NaNs);
//   MMA warps       one issuing thread per query tile.  Per KV tile j thread t issues one burst:
//                   O_t += P_t(j-1) V(j-1) with P read from tensor memory (it overwrites S in place
//                   as packed bf16) and V consumed MN-major straight from the TMA layout, then
//                   S_t(j) = Q_t K(j)^T (M=128, N=BN, fp32 accumulators in tensor memory), which
//                   overwrites P_t(j-1).  A tcgen05.mma of this size costs its issuing thread about
//                   as long as the tensor pipe needs to run it, and every wait or commit of that
//                   thread adds to it, so one thread for both tiles is the bottleneck; two threads
//                   left alone fall into step (both softmax groups then meet on the MUFU, both
//                   bursts on the tensor pipe).  The bursts therefore strictly alternate (a token
//                   passed through two barriers): one tile's products run under the other tile's
//                   softmax.  The first 64 keys of P_t V are issued outside the turn, while the
//                   softmax group is still exponentiating the other 64;
//                   With ONE query tile (head_dim 256: O takes 256 of the 512 columns) there is no
//                   other tile to fill the pipe during the softmax, but room for a second S buffer:
//                   S(j) is issued into the buffer that held P(j-2) before P(j-1) is waited for, so it
//                   runs under the softmax of tile j-1 and the softmax group never waits for S;
//   softmax groups  one warpgroup per query tile, one thread per row: tcgen05.ld brings the row of
//                   S into registers (no shuffles), running max / sum, exp2, P back to tensor
//                   memory, O rescaled in tensor memory only when the running max moved by more
//                   than 2^8 (the stale max is carried exactly through P and the row sum), and the
//                   epilogue O / l -> bf16 -> global.
// Every barrier is used round after round across items; each role keeps its own counters and derives
// the parity it waits for from them.  Every mbarrier wait is bounded; a wait that gives up poisons
// the CTA, which then drains (and stops taking items).
//
// Roofline: tensor-bound, 4 * D flops per (query, key) pair per head.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

#include <type_traits>

namespace mvb {

struct PrefillParams {
  const int32_t* cu_q;
  const int32_t* cu_k;
  const int32_t* block_table;   // nullptr: dense K/V
  int64_t table_stride;
  int block_size;
  int64_t kv_rows;
  int num_seqs, hq, group;
  int pair_heads;               // 1: an item's query tiles are the heads of one GQA group over the same rows
  float scale_log2;
  int window_left;
  __nv_bfloat16* out;
  int64_t out_stride;
  int* dev_status;
  // nullptr, or the launch's work as a list of num_items (sequence, query block) pairs: blockIdx.y picks the pair.
  // Without it the grid has a block index for every (sequence, query-block rank) up to the longest sequence's
  // count, and the indices past a sequence's last block cost their taker a launch-control round trip each.
  const int32_t* items;
  int num_items;
};

// barrier slots
// P is published in 64-key halves (slot B_PFULL + 2 * tile + half) so the PV product of the first
// half starts while the second half is still being exponentiated.  B_TURN + t: tile t's issuing thread
// may issue its next burst.
enum : int { B_QFULL = 0, B_KFULL = 2, B_VFULL = 4, B_KFREE = 6, B_VFREE = 8, B_SFULL = 10, B_PFULL = 12,
             B_TURN = 28, B_ODONE = 16, B_OFREE = 18, B_VFIXED = 20, B_QFREE = 22, B_ITEM_FULL = 23, B_ITEM_FREE = 25,
             B_CLC = 27, B_PVDONE = 30, B_COUNT = 31 };

template <int D, int BN, int NQ>
struct PrefillCfg {
  static constexpr int THREADS = NQ * 128 + 32 + NQ * 32;   // softmax groups, producer warp, one MMA warp per query tile
  static constexpr int Q_BYTES = 128 * D * 2;          // one query tile
  static constexpr int KV_BYTES = BN * D * 2;          // one K (or V) tile
  static constexpr int HALF_Q = 128 * 128;             // bytes of one 64-column half of a Q tile
  static constexpr int HALF_KV = BN * 128;             // bytes of one 64-column half of K / V
  // after the tiles: barriers, the tensor-memory address, the failure flag, two item slots and the
  // launch-control response
  static constexpr int CTRL_BYTES = 512;
  static constexpr int OFF_TMEM_SLOT = B_COUNT * 8, OFF_FAIL = OFF_TMEM_SLOT + 4, OFF_ITEMS = 256, OFF_CLC = 352;
  static constexpr int STAGE_BYTES = NQ * 4 * 4096;     // a 32-row x 128-byte output staging tile per softmax warp
  static constexpr int SMEM = NQ * Q_BYTES + 4 * KV_BYTES + 1024 /*align*/ + CTRL_BYTES + STAGE_BYTES;
  // With one query tile there is room for a second S buffer: the S product of KV tile j + 1 is then issued before
  // P of tile j is waited for and runs under that tile's softmax (with two tiles the other tile's products do).
  static constexpr int S_BUFS = NQ == 1 ? 2 : 1;
  static constexpr int TMEM_COLS = NQ * (S_BUFS * BN + D) <= 256 ? 256 : 512;   // power of two
  static constexpr int S_COL = 0;                      // S_t, buffer b at S_COL + (t * S_BUFS + b) * BN (P aliases its first BN/2 columns)
  static constexpr int O_COL = NQ * S_BUFS * BN;       // O_t at O_COL + t * D
  static_assert(NQ * (S_BUFS * BN + D) <= 512, "tensor memory budget");
  static_assert(S_BUFS == 1 || BN == 64, "the two-buffer form publishes P once per 64-key tile");
  static_assert(BN % 64 == 0, "P is written in 64-key halves");
  static_assert(OFF_FAIL + 4 <= OFF_ITEMS && OFF_CLC + 16 <= CTRL_BYTES, "control block layout");
};

// What every role derives from an item's block index.
template <int BN, int NQ, bool LIST>
struct PrefillItem {
  int s, q0, k0, k_len, row0, kvh;
  int rows[NQ], pf[NQ], pl[NQ], jlo[NQ], jhi[NQ], roff[NQ], head[NQ];
  int j_lo, j_hi, n_it;
  bool empty;                                          // block index past the sequence's last query block

  // grid = (heads or head pairs, sequences, query-block rank counted from the END of the sequence):
  // indices are handed out x-fastest, so every sequence's last query block (the one with the most
  // keys) is worked on before any second-to-last one, which keeps the tail of the launch short.
  // With an item list: grid = (heads or head pairs, items), the list's order is the order of the work.
  // what the producer hands on with a listed item, so that the other roles read no global memory for it
  int seq_in, qb_in, q_begin_in, q_end_in, k_begin_in, k_end_in;

  __device__ __forceinline__ void init(const PrefillParams& p, int bx, int by, int bz) {
    int s_ = by, qb_ = 0;
    if constexpr (LIST) {
      s_ = p.items[2 * by];
      qb_ = p.items[2 * by + 1];
      if (s_ < 0 || s_ >= p.num_seqs) { s_ = 0; qb_ = -1; }      // a bad entry comes out as an empty item
    }
    init_from(p, bx, bz, s_, qb_, p.cu_q[s_], p.cu_q[s_ + 1], p.cu_k[s_], p.cu_k[s_ + 1]);
  }

  __device__ __forceinline__ void init_from(const PrefillParams& p, int bx, int bz, int s_, int listed_qb, int q_begin,
                                            int q_end, int k_begin, int k_end) {
    seq_in = s_; qb_in = listed_qb; q_begin_in = q_begin; q_end_in = q_end; k_begin_in = k_begin; k_end_in = k_end;
    s = s_;
    const bool pair = p.pair_heads != 0;
    // The NQ query tiles of an item are either NQ heads of one GQA group over the same 128 rows (each
    // K/V tile loaded once serves them all: half the K/V traffic per flop) or, without a group to
    // share, NQ consecutive 128-row tiles of one head.
    const int qh0 = pair ? bx * NQ : bx;
    kvh = qh0 / p.group;
    const int rows_per_item = pair ? 128 : 128 * NQ;
    q0 = q_begin;
    k0 = k_begin;
    const int q_len = q_end - q0;
    k_len = k_end - k0;
    const int n_qb = (q_len + rows_per_item - 1) / rows_per_item;
    const int qb = LIST ? listed_qb : n_qb - 1 - bz;
    empty = qb < 0 || qb >= n_qb;
    row0 = qb * rows_per_item;
    const int shift = k_len - q_len;                   // position of query row 0
    j_lo = 0x7fffffff;
    j_hi = -1;
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
      roff[t] = pair ? 0 : 128 * t;
      head[t] = pair ? qh0 + t : qh0;
      rows[t] = empty ? 0 : max(0, min(128, q_len - row0 - roff[t]));
      pf[t] = shift + row0 + roff[t];
      pl[t] = pf[t] + rows[t] - 1;
      jlo[t] = p.window_left >= 0 ? max(0, pf[t] - p.window_left) / BN : 0;
      jhi[t] = rows[t] > 0 ? pl[t] / BN : -1;
      if (rows[t] > 0) { j_lo = min(j_lo, jlo[t]); j_hi = max(j_hi, jhi[t]); }
    }
    n_it = j_hi - j_lo + 1;
    if (n_it <= 0) empty = true;
  }
};

// LIST: the work comes as a list of (sequence, query block) pairs (PrefillParams::items) instead of a 3-D grid; a
// kernel of its own, so that the grid form carries none of the list's code.
template <int D, int BN, int NQ, bool LIST>
__global__ void __launch_bounds__(PrefillCfg<D, BN, NQ>::THREADS, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
  using C = PrefillCfg<D, BN, NQ>;
  using Item = PrefillItem<BN, NQ, LIST>;
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, BN, false, false);
  constexpr uint32_t IDESC_O = umma_idesc_bf16(128, D, false, true);
  extern __shared__ uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  {
    // a CTA whose own index is past its sequence's last query block has nothing to set up; the indices
    // still pending are taken by the CTAs that are at work
    Item own;
    own.init(p, blockIdx.x, blockIdx.y, blockIdx.z);
    if (own.empty) return;                                    // CTA-uniform
  }

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base;                                  // NQ tiles
  const uint32_t k_s = q_s + NQ * C::Q_BYTES;                 // 2 stages
  const uint32_t v_s = k_s + 2 * C::KV_BYTES;                 // 2 stages
  uint8_t* ctrl = base_ptr + NQ * C::Q_BYTES + 4 * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + C::OFF_TMEM_SLOT);
  volatile uint32_t* fail_flag = reinterpret_cast<uint32_t*>(ctrl + C::OFF_FAIL);
  volatile int4* items = reinterpret_cast<volatile int4*>(ctrl + C::OFF_ITEMS);   // slots 0-1: {x, y, z, valid}; list form: 2-5 hold each slot's (sequence, block, q bounds), (k bounds)
  const uint32_t clc_resp = smem_u32(ctrl + C::OFF_CLC);
  const uint32_t stage_s = smem_u32(ctrl + C::CTRL_BYTES);

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) {
      uint32_t count = 1u;
      if (i >= B_PFULL && i < B_PFULL + 4) count = 4u;          // one lane per softmax warp
      if (i >= B_OFREE && i < B_OFREE + 2) count = 4u;
      if ((i >= B_KFREE && i < B_KFREE + 4) || i == B_QFREE) count = NQ;   // every MMA thread releases every stage
      if (i >= B_ITEM_FREE && i < B_ITEM_FREE + 2) count = NQ + NQ * 128u;
      mbar_init(&bars[i], count);
    }
    *fail_flag = 0;
    fence_mbar_init();
    mbar_arrive(&bars[B_TURN + 0]);                           // the first burst is tile 0's
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
    if (mbar_try_wait(&bars[slot], parity)) return true;
    return mbar_wait_or_fail(&bars[slot], parity, fail_flag, p.dev_status, where);
  };
  // The consumer side of the item ring: false at the end of the work (or on failure).
  auto next_item = [&](uint32_t n, Item& item) -> bool {
    const int slot = n & 1;
    if (!wait(B_ITEM_FULL + slot, (n >> 1) & 1, 900)) return false;
    const int x = items[slot].x, y = items[slot].y, z = items[slot].z, valid = items[slot].w;
    if constexpr (LIST) {
      const int4 a = const_cast<const int4&>(const_cast<volatile int4&>(items[2 + 2 * slot]));
      const int4 b = const_cast<const int4&>(const_cast<volatile int4&>(items[3 + 2 * slot]));
      mbar_arrive(&bars[B_ITEM_FREE + slot]);
      if (!valid) return false;
      item.init_from(p, x, z, a.x, a.y, a.z, a.w, b.x, b.y);
      return true;
    }
    mbar_arrive(&bars[B_ITEM_FREE + slot]);
    if (!valid) return false;
    item.init(p, x, y, z);
    return true;
  };

  if (warp == NQ * 4) {
    // ============================ producer warp ======================================================
    // All lanes walk the items together (the zero fill is warp-wide); lane 0 owns barriers and TMA.
    Item item;
    int bx = blockIdx.x, by = blockIdx.y, bz = blockIdx.z;
    uint32_t n_pub = 0, n_clc = 0, g = 0;                     // items published, responses read, KV tiles loaded
    uint32_t k_issued = 0, v_issued = 0;                      // lane 0: K / V tile loads handed to TMA
    bool clc_pending = false;                                 // lane 0: a request whose response has not been read
    bool ok = true, have = true;
    if (lane == 0) { tma_prefetch_desc(&q_map); tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map); }
    auto publish = [&](int x, int y, int z, int valid) {      // lane 0
      const int slot = n_pub & 1;
      if (n_pub >= 2) ok = wait(B_ITEM_FREE + slot, ((n_pub >> 1) - 1) & 1, 910);
      if (ok) {
        items[slot].x = x; items[slot].y = y; items[slot].z = z; items[slot].w = valid;
        if constexpr (LIST) {
          items[2 + 2 * slot].x = item.seq_in; items[2 + 2 * slot].y = item.qb_in;
          items[2 + 2 * slot].z = item.q_begin_in; items[2 + 2 * slot].w = item.q_end_in;
          items[3 + 2 * slot].x = item.k_begin_in; items[3 + 2 * slot].y = item.k_end_in;
        }
        mbar_arrive(&bars[B_ITEM_FULL + slot]);
      }
    };
    auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint64_t* bar, int z) {
      mbar_arrive_expect_tx(bar, C::KV_BYTES);
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst + h * C::HALF_KV), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(h * 64),
              "r"(item.kvh), "r"(z) : "memory");
      }
    };
    auto kv_row = [&](int j) -> int {                         // tensor-map row of KV tile j of this sequence
      const int tok = j * BN;
      if (p.block_table == nullptr) return item.k0 + tok;
      const int blk = p.block_table[item.s * p.table_stride + tok / p.block_size];
      if (blk < 0 || static_cast<int64_t>(blk + 1) * p.block_size > p.kv_rows) {
        report(p.dev_status, kDevBadBlock, item.s);
        return -BN;                                           // fully out of range: zero fill
      }
      return blk * p.block_size + tok % p.block_size;
    };
    while (ok && have) {
      item.init(p, bx, by, bz);
      if (lane == 0) {
        if (!item.empty) publish(bx, by, bz, 1);
        if (ok) {                                             // ask for the next index while this one is worked on
          fence_proxy_async();                                // the response slot was last read with ordinary loads
          mbar_arrive_expect_tx(&bars[B_CLC], 16);
          clc_try_cancel(clc_resp, &bars[B_CLC]);
          clc_pending = true;
        }
      }
      if (!item.empty) {
        // The Q tiles are single-buffered: every S product of the previous item must have read them.
        // They are asked for after the item's first K and V tiles, which do not have to wait for that.
        auto load_q = [&]() {                                 // lane 0
          if (n_pub >= 2) ok = wait(B_QFREE, n_pub & 1, 920);
#pragma unroll
          for (int t = 0; t < NQ; ++t) {
            if (!ok || item.rows[t] <= 0) continue;
            mbar_arrive_expect_tx(&bars[B_QFULL + t], C::Q_BYTES);
#pragma unroll
            for (int h = 0; h < D / 64; ++h) {
              asm volatile(
                  "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                  ::"r"(q_s + t * C::Q_BYTES + h * C::HALF_Q), "l"(reinterpret_cast<uint64_t>(&q_map)),
                    "r"(smem_u32(&bars[B_QFULL + t])), "r"(h * 64), "r"(item.head[t]),
                    "r"(item.q0 + item.row0 + item.roff[t]) : "memory");
            }
          }
        };
        ++n_pub;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        for (int it = 0; it < item.n_it && ok; ++it, ++g) {
          const int st = g & 1, j = item.j_lo + it;
          const uint32_t ring_parity = (g >> 1) & 1;
          if (lane == 0) {
            const int z = kv_row(j);
            if (g >= 2) ok = wait(B_KFREE + st, ring_parity ^ 1, 100);
            if (ok) { load_tile(&k_map, k_s + st * C::KV_BYTES, &bars[B_KFULL + st], z); ++k_issued; }
            if (ok && g >= 2) ok = wait(B_VFREE + st, ring_parity ^ 1, 200);
            if (ok) { load_tile(&v_map, v_s + st * C::KV_BYTES, &bars[B_VFULL + st], z); ++v_issued; }
            if (ok && it == 0) load_q();
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          const int valid = item.k_len - j * BN;
          if (ok && valid < BN) {                             // last, partial tile: zero V rows past the end
            ok = __all_sync(0xffffffffu, wait(B_VFULL + st, ring_parity, 300));
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
              if (lane == 0) mbar_arrive(&bars[B_VFIXED + st]);
            }
          }
        }
      }
      // the next index (or the end of the work)
      int nx = 0, ny = 0, nz = 0, more = 0;
      if (lane == 0 && ok) {
        ok = wait(B_CLC, n_clc & 1, 930);
        if (ok) {
          clc_pending = false;
          more = clc_query(clc_resp, nx, ny, nz) ? 1 : 0;
          if (more && (nx >= static_cast<int>(gridDim.x) || ny >= static_cast<int>(gridDim.y) ||
                       nz >= static_cast<int>(gridDim.z))) {
            report(p.dev_status, kDevWaitTimeout, 931);       // an index outside the grid: stop taking items
            *fail_flag = 1;
            ok = false;
          }
        }
      }
      ++n_clc;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      have = __shfl_sync(0xffffffffu, more, 0) != 0;
      bx = __shfl_sync(0xffffffffu, nx, 0);
      by = __shfl_sync(0xffffffffu, ny, 0);
      bz = __shfl_sync(0xffffffffu, nz, 0);
    }
    if (lane == 0 && ok) publish(0, 0, 0, 0);                 // end of the work
    if (lane == 0 && !ok) {
      // poisoned: nothing asynchronous may still be writing this CTA's shared memory when it ends
      if (clc_pending) mbar_wait(&bars[B_CLC], n_clc & 1);
      for (uint32_t back = 1; back <= 2; ++back) {
        if (k_issued >= back) mbar_wait(&bars[B_KFULL + ((k_issued - back) & 1)], ((k_issued - back) >> 1) & 1);
        if (v_issued >= back) mbar_wait(&bars[B_VFULL + ((v_issued - back) & 1)], ((v_issued - back) >> 1) & 1);
      }
    }
  } else if (warp >= NQ * 4 + 1) {
    // ============================ MMA warps: one issuing thread per query tile =========================
    // Thread t issues, per KV tile j, one burst: O_t += P_t(j-1) V(j-1), then S_t(j) = Q_t K(j)^T.  The
    // bursts of the two threads strictly alternate (B_TURN).  Both threads walk every KV tile of every
    // item and release every ring stage, also in steps their tile sits out.
    const int t = warp - (NQ * 4 + 1);
    if (lane == 0) {
      bool ok = true;
      const uint64_t q_desc = umma_desc_sw128(q_s + t * C::Q_BYTES, 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(k_s, 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(v_s, C::HALF_KV, 1024);
      const uint32_t s_tm = tmem + C::S_COL + t * C::S_BUFS * BN, o_tm = tmem + C::O_COL + t * D;
      uint32_t g = 0;                                         // KV tiles walked (ring position)
      uint32_t n_pv = 0;                                      // PV products issued (P parity)
      uint32_t n_act = 0;                                     // items in which this tile had rows (Q / O parity)
      uint32_t n_burst = 0;                                   // bursts issued (turn parity)
      uint32_t fix_parity = 0;                                // bit st: parity of the next V fix-up on ring stage st
      auto ready = [&](int slot, uint32_t parity, int where) -> bool {
        return mbar_try_wait(&bars[slot], parity) ? true : wait(slot, parity, where);
      };
      Item item;
      for (uint32_t n_item = 0; ok && next_item(n_item, item); ++n_item) {
        int rows = item.rows[0], jlo = item.jlo[0], jhi = item.jhi[0];
#pragma unroll
        for (int u = 1; u < NQ; ++u)
          if (t == u) { rows = item.rows[u]; jlo = item.jlo[u]; jhi = item.jhi[u]; }
        if (rows <= 0) { jlo = 1; jhi = 0; }                  // this tile sits the item out (it still walks the ring)
        const int j_partial = item.k_len / BN;                // first KV tile with rows past the end
        const int n_it = item.n_it, j_lo = item.j_lo;
        if constexpr (NQ == 1) {
          // One tile, two S buffers.  Step `it`: S of KV tile j into the buffer that held P of tile j - 2 (its PV
          // product was issued before, and the pipe runs in order), then, once the softmax group has published
          // P of tile j - 1, the PV product of that tile; one extra step for the last PV.
          for (int it = 0; it <= n_it && ok; ++it) {
            const int j = j_lo + it;
            const bool body = it < n_it;
            const int st = g & 1, stp = (g - 1) & 1;
            if (body) {
              ok = ready(B_KFULL + st, (g >> 1) & 1, 600);
              if (ok && j == jlo) ok = ready(B_QFULL + 0, n_act & 1, 610);
              if (!ok) break;
              tc_fence_after();
              const uint32_t buf = n_burst & 1;                // (n_burst counts the S products here)
              const uint64_t kd = k_desc0 + ((st * C::KV_BYTES) >> 4);
#pragma unroll
              for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t qo = ((ks >> 2) * C::HALF_Q + (ks & 3) * 32) >> 4, ko = ((ks >> 2) * C::HALF_KV + (ks & 3) * 32) >> 4;
                umma_bf16_ss(s_tm + buf * BN, q_desc + qo, kd + ko, IDESC_S, ks > 0);
              }
              umma_commit(&bars[B_SFULL + buf]);
              ++n_burst;
              umma_commit(&bars[B_KFREE + st]);
              if (it == n_it - 1) umma_commit(&bars[B_QFREE]);
            }
            if (it >= 1) {
              ok = ready(B_VFULL + stp, ((g - 1) >> 1) & 1, 400);
              if (ok && j - 1 >= j_partial) ok = ready(B_VFIXED + stp, (fix_parity >> stp) & 1, 450);
              uint32_t first = 1u;
              if (ok && j - 1 == jlo) {
                first = 0u;
                if (n_act > 0) ok = ready(B_OFREE + 0, (n_act - 1) & 1, 460);
              }
              const uint32_t pbuf = n_pv & 1;
              if (ok) ok = ready(B_PFULL + pbuf, (n_pv >> 1) & 1, 500);
              if (!ok) break;
              tc_fence_after();
              const uint64_t vd = v_desc0 + ((stp * C::KV_BYTES) >> 4);
#pragma unroll
              for (int ks = 0; ks < BN / 16; ++ks)
                umma_bf16_ts(o_tm, s_tm + pbuf * BN + ks * 8, vd + ((ks * 2048) >> 4), IDESC_O, ks > 0 ? 1u : first);
              umma_commit(&bars[B_PVDONE]);                   // a rescale of O waits for it
              if (j - 1 == jhi) umma_commit(&bars[B_ODONE + 0]);
              ++n_pv;
              umma_commit(&bars[B_VFREE + stp]);
            }
            if (body) ++g;
          }
        } else
        // step `it`: PV of KV tile j - 1, then S of tile j; one extra step for the last PV
        for (int it = 0; it <= n_it && ok; ++it) {
          const int j = j_lo + it;
          const bool body = it < n_it;
          const bool act_s = body && j >= jlo && j <= jhi;
          const bool act_pv = it >= 1 && j - 1 >= jlo && j - 1 <= jhi;
          const int st = g & 1, stp = (g - 1) & 1;            // ring stages of tile j and of tile j - 1
          // everything the burst needs, then the turn
          if (body) ok = ready(B_KFULL + st, (g >> 1) & 1, 600);
          if (ok && act_s && j == jlo) ok = ready(B_QFULL + t, n_act & 1, 610);
          if (ok && it >= 1) {
            ok = ready(B_VFULL + stp, ((g - 1) >> 1) & 1, 400);
            if (ok && j - 1 >= j_partial) ok = ready(B_VFIXED + stp, (fix_parity >> stp) & 1, 450);
          }
          uint32_t first = 1u;
          if (ok && act_pv) {
            if (j - 1 == jlo) {
              first = 0u;                                     // an item's first product overwrites O_t: the previous epilogue has read it
              if (n_act > 0) ok = ready(B_OFREE + t, (n_act - 1) & 1, 460);
            }
            if (ok) ok = ready(B_PFULL + 2 * t, n_pv & 1, 500);
          }
          if (!ok) break;
          tc_fence_after();
          const uint64_t vd = v_desc0 + ((stp * C::KV_BYTES) >> 4);
          if (act_pv) {                                       // O_t (+)= P_t . V, first 64 keys: under the softmax of the other 64
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_bf16_ts(o_tm, s_tm + ks * 8, vd + ((ks * 2048) >> 4), IDESC_O, ks > 0 ? 1u : first);
            if constexpr (BN > 64) {
              ok = ready(B_PFULL + 2 * t + 1, n_pv & 1, 501);
            }
          }
          if constexpr (NQ > 1) {
            if (ok) ok = ready(B_TURN + t, n_burst & 1, 620);
          }
          if (!ok) break;
          tc_fence_after();
          if (act_pv) {
            if constexpr (BN > 64) {
#pragma unroll
              for (int ks = 4; ks < BN / 16; ++ks)
                umma_bf16_ts(o_tm, s_tm + ks * 8, vd + ((ks * 2048) >> 4), IDESC_O, 1u);
            }
            if (j - 1 == jhi) umma_commit(&bars[B_ODONE + t]);  // the item's last product: the epilogue waits for it
            ++n_pv;
          }
          if (act_s) {                                        // S_t = Q_t . K^T
            const uint64_t kd = k_desc0 + ((st * C::KV_BYTES) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint32_t qo = ((ks >> 2) * C::HALF_Q + (ks & 3) * 32) >> 4, ko = ((ks >> 2) * C::HALF_KV + (ks & 3) * 32) >> 4;
              umma_bf16_ss(s_tm, q_desc + qo, kd + ko, IDESC_S, ks > 0);
            }
            umma_commit(&bars[B_SFULL + t]);
          }
          if constexpr (NQ > 1) mbar_arrive(&bars[B_TURN + (t ^ 1)]);
          if (it >= 1) umma_commit(&bars[B_VFREE + stp]);
          if (body) {
            umma_commit(&bars[B_KFREE + st]);
            if (it == n_it - 1) umma_commit(&bars[B_QFREE]);  // the item's last S product has been issued
          }
          ++n_burst;
          if (body) ++g;
        }
        // a partial tile is an item's last one: its fix-up, on the ring stage just left, has been consumed
        if (item.j_hi >= j_partial) fix_parity ^= 1u << ((g - 1) & 1);
        if (rows > 0) ++n_act;
      }
    }
    __syncwarp();
  } else {
    // ============================ softmax warpgroup of query tile t ==================================
    const int t = warp >> 2;
    const int row = tid & 127;                                // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_base = lane_addr + C::S_COL + t * C::S_BUFS * BN;
    const uint32_t o_addr = lane_addr + C::O_COL + t * D;
    uint32_t n_s = 0, n_epi = 0;                              // S tiles consumed (S / P parity), epilogues done (O parity)
    bool ok = true;
    Item item;
    for (uint32_t n_item = 0; ok && next_item(n_item, item); ++n_item) {
      // this group's tile, picked with selects so the item stays in registers
      int rows_me = item.rows[0], pf_me = item.pf[0], pl_me = item.pl[0], jlo_me = item.jlo[0], jhi_me = item.jhi[0],
          roff_me = item.roff[0], head_me = item.head[0];
#pragma unroll
      for (int u = 1; u < NQ; ++u)
        if (t == u) {
          rows_me = item.rows[u]; pf_me = item.pf[u]; pl_me = item.pl[u]; jlo_me = item.jlo[u]; jhi_me = item.jhi[u];
          roff_me = item.roff[u]; head_me = item.head[u];
        }
      if (rows_me <= 0) continue;
      const int my_pos = pf_me + row;                    // absolute position of this row's query
      const int hi_key = my_pos;
      const int lo_key = p.window_left >= 0 ? my_pos - p.window_left : 0;
      float m_run = -INFINITY, l_run = 0.f;
      const int n_itt = jhi_me - jlo_me + 1;
      for (int itt = 0; itt < n_itt && ok; ++itt, ++n_s) {
        const int j = jlo_me + itt, col0 = j * BN;
        const uint32_t sbuf = C::S_BUFS == 2 ? (n_s & 1) : 0u;    // which S buffer this tile is in
        const uint32_t s_addr = s_base + sbuf * BN;
        ok = C::S_BUFS == 2 ? wait(B_SFULL + sbuf, (n_s >> 1) & 1, 700) : wait(B_SFULL + t, n_s & 1, 700);
        if (!ok) break;
        tc_fence_after();
        // Visible keys of this row inside the tile: [vis_lo, vis_hi] relative to col0.  The rows of a
        // warp are consecutive, so a 32-key chunk is classified once per warp: visible to all 32 rows
        // (no mask arithmetic), to none (not loaded at all; P = 0), or mixed (per-element mask bits).
        const int vis_hi = hi_key - col0;
        const int vis_lo = p.window_left >= 0 ? lo_key - col0 : -0x40000000;
        const int w_hi = vis_hi - lane, w_lo = vis_lo - lane;     // bounds of the warp's first row; its last row: + 31
        auto chunk_class = [&](int cb) -> int {
          if (cb + 31 <= w_hi && cb >= w_lo + 31) return 0;
          if (cb > w_hi + 31 || cb + 31 < w_lo) return 2;
          return 1;
        };
        auto visible_bits = [&](int cb) -> uint32_t {             // bit i: key cb + i is visible to this row
          const int lo = max(vis_lo - cb, 0), hi = min(vis_hi - cb, 31);
          return hi < lo ? 0u : ((0xffffffffu >> (31 - hi)) & (0xffffffffu << lo));
        };
        // Two bodies.  Tiles that every row of the warp sees completely (the common case) bring the
        // thread's whole row of S into registers once - one wait for all the loads, so their latency is
        // paid once per tile - and keep it there for both passes, with no mask code at all.  The other
        // tiles (the diagonal, the window's edge) go chunk by chunk and read S twice.
        float sum0 = 0.f, sum1 = 0.f, alpha = 1.f, m_use = m_run;
        constexpr int NCH = BN / 32;
        // new running maximum (lazy: keep the old one unless the tile's is more than 2^8 larger) and the
        // rescale of O that goes with it; S_t(itt) complete implies PV_t(itt-1) complete (one thread
        // issues both, in order), so O is ours
        auto new_max = [&](float tile_max) {
          tile_max *= p.scale_log2;                           // scale > 0, so max commutes with it
          if (tile_max > m_run + 8.f || (m_run == -INFINITY && tile_max > -INFINITY)) {
            m_use = tile_max;
            alpha = fast_exp2(m_run - m_use);                 // m_run = -inf -> 0
          }
          if (itt > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
            if constexpr (C::S_BUFS == 2) {
              // this tile's S was issued BEFORE the PV product of the previous tile (the n_s-th of this group,
              // counted from 1): O is ours only when that product has completed
              ok = wait(B_PVDONE, (n_s - 1) & 1, 710);
              tc_fence_after();
            }
#pragma unroll 1
            for (int c = 0; c < D / 16; ++c) {                // rare: small chunks, to stay short of registers
              uint32_t r[16];
              tmem_ld_32x16(o_addr + c * 16, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x16(o_addr + c * 16, r);
            }
          }
        };
        // P = exp2(S * scale - m) as packed bf16 over the first BN/2 columns of S (keys c*32 + i, i+1 ->
        // word c*16 + i/2), written per 32 keys and published per 64 by one lane per warp
        auto publish_p = [&](int c, const uint32_t (&pk)[16]) {
          tmem_st_32x16(s_addr + c * 16, pk);
          if (c & 1) {
            tmem_wait_st();                                   // warp-wide: every lane's words are in tensor memory
            if (lane == 0) {
              tc_fence_before();
              mbar_arrive(&bars[C::S_BUFS == 2 ? B_PFULL + sbuf : B_PFULL + 2 * t + (c >> 1)]);
            }
          }
        };
        if (w_hi >= BN - 1 && w_lo + 31 <= 0) {
          uint32_t sreg[NCH][32];
#pragma unroll
          for (int c = 0; c < NCH; ++c) tmem_ld_32x32(s_addr + c * 32, sreg[c]);
          tmem_wait_ld();
          float max0 = -INFINITY, max1 = -INFINITY;
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              max0 = fmax3(max0, __uint_as_float(sreg[c][i]), __uint_as_float(sreg[c][i + 1]));
              max1 = fmax3(max1, __uint_as_float(sreg[c][i + 2]), __uint_as_float(sreg[c][i + 3]));
            }
          new_max(fmaxf(max0, max1));
          const float m_safe = m_use == -INFINITY ? 0.f : m_use;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(sreg[c][i]), p.scale_log2, -m_safe));
              const float e1 = fast_exp2(fmaf(__uint_as_float(sreg[c][i + 1]), p.scale_log2, -m_safe));
              sum0 += e0; sum1 += e1;
              pk[i >> 1] = pack_bf16(e0, e1);
            }
            publish_p(c, pk);
          }
        } else {
          // chunks every row of the warp sees completely run the plain code here too
          float tile_max = -INFINITY;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            const int cl = chunk_class(c * 32);
            if (cl == 2) continue;
            uint32_t r[32];
            tmem_ld_32x32(s_addr + c * 32, r);
            tmem_wait_ld();
            if (cl == 0) {
              float max0 = -INFINITY, max1 = -INFINITY;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                max0 = fmax3(max0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                max1 = fmax3(max1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
              }
              tile_max = fmax3(tile_max, max0, max1);
            } else {
              const uint32_t bits = visible_bits(c * 32);
#pragma unroll
              for (int i = 0; i < 32; ++i)
                tile_max = fmaxf(tile_max, (bits >> i) & 1u ? __uint_as_float(r[i]) : -INFINITY);
            }
          }
          new_max(tile_max);
          const float m_safe = m_use == -INFINITY ? 0.f : m_use;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            uint32_t pk[16];
            const int cl = chunk_class(c * 32);
            if (cl == 2) {
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = 0u;
            } else {
              uint32_t r[32];
              tmem_ld_32x32(s_addr + c * 32, r);
              tmem_wait_ld();
              if (cl == 1) {
                const uint32_t bits = visible_bits(c * 32);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (!((bits >> i) & 1u)) r[i] = 0xff800000u;  // -inf
              }
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float e0 = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_safe));
                const float e1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_safe));
                sum0 += e0; sum1 += e1;
                pk[i >> 1] = pack_bf16(e0, e1);
              }
            }
            publish_p(c, pk);
          }
        }
        l_run = l_run * alpha + (sum0 + sum1);
        m_run = m_use;
      }
      // ---- epilogue: while it runs, the other roles are already at work on the next item ------------
      if (ok) ok = wait(B_ODONE + t, n_epi & 1, 800);
      ++n_epi;
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        // the whole row of O, normalised, as bf16 pairs in registers; then O_t belongs to the next item
        uint32_t packed[D / 2];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[c * 16 + i] = pack_bf16(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
        }
        if (lane == 0) {                                      // the wait above is warp-wide
          tc_fence_before();
          mbar_arrive(&bars[B_OFREE + t]);
        }
        // A thread owns a row, so storing from registers would touch 32 lines per instruction.  Each
        // warp turns its 32 rows through a 4 KB staging tile (16-byte units XOR-swizzled by the row,
        // conflict-free both ways) and writes whole 128-byte lines, 64 columns at a time.
        const uint32_t stage = stage_s + warp * 4096;
        const int wrow0 = (warp & 3) * 32;
        __nv_bfloat16* obase = p.out + (static_cast<int64_t>(item.q0) + item.row0 + roff_me + wrow0) * p.out_stride +
                               static_cast<int64_t>(head_me) * D;
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + ((u ^ (lane & 7)) << 4)),
                         "r"(packed[h * 32 + u * 4]), "r"(packed[h * 32 + u * 4 + 1]), "r"(packed[h * 32 + u * 4 + 2]),
                         "r"(packed[h * 32 + u * 4 + 3]) : "memory");
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3), un = lane & 7;
            uint4 w;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                         : "r"(stage + rr * 128 + ((un ^ (rr & 7)) << 4)) : "memory");
            if (wrow0 + rr < rows_me)
              *reinterpret_cast<uint4*>(obase + static_cast<int64_t>(rr) * p.out_stride + h * 64 + un * 8) = w;
          }
          __syncwarp();
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

template <int D, int BN, int NQ, bool LIST>
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
  using KernelTag = std::integral_constant<int, D * 8 + NQ * 2 + (LIST ? 1 : 0)>;   // one opt-in record per kernel
  rc = opt_in_dynamic_smem<KernelTag>(reinterpret_cast<const void*>(&prefill_attn_kernel<D, BN, NQ, LIST>), C::SMEM);
  if (rc != kOk) return rc;
  PrefillParams pp = p;
  pp.pair_heads = (NQ > 1 && p.group % NQ == 0) ? 1 : 0;
  const int rows_per_cta = pp.pair_heads ? 128 : 128 * NQ;
  dim3 grid(pp.pair_heads ? p.hq / NQ : p.hq, p.num_seqs, (max_seqlen_q + rows_per_cta - 1) / rows_per_cta);
  if (grid.z > 65535) return kUnsupportedShape;
  if constexpr (LIST) {
    if (p.num_items > 65535) return kUnsupportedShape;
    grid.y = p.num_items;
    grid.z = 1;
  }
  prefill_attn_kernel<D, BN, NQ, LIST><<<grid, C::THREADS, C::SMEM, stream>>>(qm, km, vm, pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace mvb

// rows of q that one work item covers: the two query tiles of an item are two heads of a GQA group over the same 128
// rows when the group allows it, else two consecutive 128-row tiles of one head (head_dim 128); one tile for head_dim 256
static int prefill_item_rows(int num_q_heads, int num_kv_heads, int head_dim) {
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return mvb::kInvalidArgument;
  if (head_dim == 256) return 128;
  if (head_dim != 128) return mvb::kUnsupportedShape;
  return ((num_q_heads / num_kv_heads) % 2 == 0) ? 128 : 256;
}

static int prefill_attn_impl(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride, const void* v,
                             int64_t v_row_stride, int64_t kv_rows, const int32_t* cu_seqlens_q,
                             const int32_t* cu_seqlens_k, const int32_t* block_table, int64_t table_stride,
                             int block_size, int num_seqs, int total_q, int max_seqlen_q, int num_q_heads,
                             int num_kv_heads, int head_dim, float scale, int window_left, void* out,
                             int64_t out_row_stride, const int32_t* items, int num_items, int32_t* dev_status,
                             void* stream) {
  using namespace mvb;
  if (!q || !k || !v || !cu_seqlens_q || !cu_seqlens_k || !out) return kInvalidArgument;
  if (num_seqs <= 0 || total_q < 0 || max_seqlen_q < 0 || kv_rows <= 0) return kInvalidArgument;
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return kInvalidArgument;
  if (head_dim != 128 && head_dim != 256) return kUnsupportedShape;
  if (block_table != nullptr && block_size <= 0) return kInvalidArgument;
  if (kv_rows > 0x7fffffffLL || num_seqs > 65535 || num_q_heads > 65535) return kUnsupportedShape;
  if (items != nullptr && num_items < 0) return kInvalidArgument;
  if (total_q == 0 || max_seqlen_q == 0 || (items != nullptr && num_items == 0)) return kOk;
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
  p.items = items; p.num_items = num_items;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (items != nullptr) {
    // The list form pays when the grid would be mostly empty indices (a ragged batch).  When the list fills the
    // grid - sequences of about one length - both forms take the items in the same order and the grid form,
    // which reads no list, measured 2-3 % faster: run that one (a complete list gives identical results).
    const int rows = prefill_item_rows(num_q_heads, num_kv_heads, head_dim);
    const int64_t grid_items = static_cast<int64_t>(num_seqs) * ((max_seqlen_q + rows - 1) / rows);
    if (static_cast<int64_t>(num_items) * 100 < grid_items * 85) {
      if (head_dim == 128) return launch_prefill<128, 128, 2, true>(op, p, max_seqlen_q, st);
      return launch_prefill<256, 64, 1, true>(op, p, max_seqlen_q, st);
    }
  }
  if (head_dim == 128) return launch_prefill<128, 128, 2, false>(op, p, max_seqlen_q, st);
  return launch_prefill<256, 64, 1, false>(op, p, max_seqlen_q, st);
}

extern "C" int mvb_prefill_attn(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                const void* v, int64_t v_row_stride, int64_t kv_rows,
                                const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                const int32_t* block_table, int64_t table_stride, int block_size, int num_seqs,
                                int total_q, int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                                float scale, int window_left, void* out, int64_t out_row_stride,
                                int32_t* dev_status, void* stream) {
  return prefill_attn_impl(q, q_row_stride, k, k_row_stride, v, v_row_stride, kv_rows, cu_seqlens_q, cu_seqlens_k,
                           block_table, table_stride, block_size, num_seqs, total_q, max_seqlen_q, num_q_heads,
                           num_kv_heads, head_dim, scale, window_left, out, out_row_stride, nullptr, 0, dev_status,
                           stream);
}

extern "C" int mvb_prefill_item_rows(int num_q_heads, int num_kv_heads, int head_dim) {
  return prefill_item_rows(num_q_heads, num_kv_heads, head_dim);
}

extern "C" int mvb_prefill_attn_items(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                      const void* v, int64_t v_row_stride, int64_t kv_rows,
                                      const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                      const int32_t* block_table, int64_t table_stride, int block_size, int num_seqs,
                                      int total_q, int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                                      float scale, int window_left, void* out, int64_t out_row_stride,
                                      const int32_t* items, int num_items, int32_t* dev_status, void* stream) {
  if (items == nullptr) return mvb::kInvalidArgument;
  return prefill_attn_impl(q, q_row_stride, k, k_row_stride, v, v_row_stride, kv_rows, cu_seqlens_q, cu_seqlens_k,
                           block_table, table_stride, block_size, num_seqs, total_q, max_seqlen_q, num_q_heads,
                           num_kv_heads, head_dim, scale, window_left, out, out_row_stride, items, num_items,
                           dev_status, stream);
}
