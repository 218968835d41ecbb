// Fused lm_head + greedy argmax on the tcgen05 tensor cores: token[r] = argmax_n bf16(sum_k x[r,k] * W[n,k]).
//
// The reference computes logits = lm_head(hidden) for the last token of every sequence and takes their argmax
// (minivllm/models/models/qwen3.py:215-219, layers/sampler.py:31).  For a 151 936-column vocabulary that writes
// and re-reads 300 KB of logits per row.  Here the GEMM's epilogue keeps, per row, the best (value, column) of
// the tile it just finished and folds it into one 64-bit word per row in global memory; no logits leave the SM.
//
// Work: output tiles of 128 rows x 256 vocabulary columns, K = hidden in blocks of 64.  Tile ids run rows-fastest,
// so the CTAs working at the same time share W tiles through L2 and W comes out of DRAM once.  Persistent CTAs
// (one per SM) take tiles id = blockIdx.x, + gridDim.x, ...  Roles:
//   producer warp   TMA (128-byte swizzle, no multicast): per K block one x tile [128 x 64] and one W tile
//                   [256 x 64] into a 4-stage ring;
//   MMA warp        one thread issues tcgen05.mma (M = 128, N = 256, both operands K-major from shared memory),
//                   fp32 accumulators in tensor memory, two accumulator stages so the next tile's products run
//                   under this tile's epilogue;
//   epilogue        one warpgroup, one thread per row: tcgen05.ld 32 columns at a time, round to bf16 (the value
//                   the unfused path would have stored), keep the largest with the lowest column, then one
//                   atomicMax of (order-preserving key << 32 | ~column) on the row's word.
// The last CTA to finish (a counter in the scratch) turns the words into token ids, scatters them where asked
// and clears the scratch for the next call.  Every wait is bounded.
//
// Roofline: tensor-bound for hundreds of rows (2 * rows * hidden * vocab flops), HBM-bound on W for a few
// (vocab * hidden * 2 bytes).
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

namespace mvb {

constexpr int kHeadBM = 128, kHeadBN = 256, kHeadBK = 64, kHeadStages = 4;
constexpr int kHeadThreads = 6 * 32;                   // producer, MMA, four epilogue warps
constexpr int kHeadABytes = kHeadBM * kHeadBK * 2, kHeadBBytes = kHeadBN * kHeadBK * 2;
constexpr int kHeadStageBytes = kHeadABytes + kHeadBBytes;
constexpr int kHeadSmem = kHeadStages * kHeadStageBytes + 1024 /*align*/ + 256 /*barriers*/;

struct HeadParams {
  int rows, vocab, hidden;
  int m_tiles, n_tiles;
  unsigned long long* best;          // [rows] packed (key << 32 | ~column), zero between calls
  unsigned int* done;                // CTAs finished, zero between calls
  int64_t* out;
  int64_t* scatter_table;
  const int32_t* scatter_index;
  int* dev_status;
};

enum : int { HB_FULL = 0, HB_EMPTY = kHeadStages, HB_ACC_FULL = 2 * kHeadStages, HB_ACC_EMPTY = 2 * kHeadStages + 2,
             HB_COUNT = 2 * kHeadStages + 4 };

__device__ __forceinline__ uint32_t head_sort_key(uint32_t bits16) {          // monotone in the bf16 value; -0 == +0
  if (bits16 == 0x8000u) bits16 = 0;
  return (bits16 & 0x8000u) ? (~bits16 & 0xffffu) : (bits16 | 0x8000u);
}

__global__ void __launch_bounds__(kHeadThreads, 1)
lm_head_argmax_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                      const HeadParams p) {
  constexpr uint32_t IDESC = umma_idesc_bf16(kHeadBM, kHeadBN, false, false);
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kHeadStages * kHeadStageBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + HB_COUNT);
  volatile uint32_t* fail_flag = tmem_slot + 1;
  __shared__ int is_last_s;

  if (tid == 0) {
    for (int i = 0; i < HB_COUNT; ++i) mbar_init(&bars[i], (i >= HB_ACC_EMPTY) ? 4u : 1u);   // 4 epilogue warps free an accumulator
    *fail_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {                                            // the MMA warp owns the tensor memory: 2 x 256 columns
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  auto wait = [&](int slot, uint32_t parity, int where) -> bool {
    for (int spin = 0; spin < 64; ++spin) {
      if (mbar_wait(&bars[slot], parity, 1u << 14)) return true;
      if (*fail_flag) return false;
    }
    report(p.dev_status, kDevWaitTimeout, where);
    *fail_flag = 1;
    return false;
  };
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int kblocks = p.hidden / kHeadBK;

  if (warp == 0) {
    // ============================ producer ==========================================================
    if (lane == 0) {
      tma_prefetch_desc(&x_map);
      tma_prefetch_desc(&w_map);
      uint32_t g = 0;                                         // K blocks loaded (ring position)
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++g) {
          const int st = g % kHeadStages;
          if (g >= kHeadStages) ok = wait(HB_EMPTY + st, ((g / kHeadStages) - 1) & 1, 100);
          if (!ok) break;
          const uint32_t a_dst = base + st * kHeadStageBytes, b_dst = a_dst + kHeadABytes;
          mbar_arrive_expect_tx(&bars[HB_FULL + st], kHeadStageBytes);
          // the operands are viewed as [rows, hidden / 64, 64]: box (64, 1, rows of the tile); rows past the end read as zeros
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(a_dst), "l"(reinterpret_cast<uint64_t>(&x_map)), "r"(smem_u32(&bars[HB_FULL + st])), "r"(0), "r"(kb),
                "r"(mt * kHeadBM) : "memory");
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(b_dst), "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(smem_u32(&bars[HB_FULL + st])), "r"(0), "r"(kb),
                "r"(nt * kHeadBN) : "memory");
        }
      }
      if (!ok) {                                              // nothing may still be writing this CTA's shared memory when it ends
        for (uint32_t back = 1; back <= kHeadStages && back <= g; ++back)
          mbar_wait(&bars[HB_FULL + ((g - back) % kHeadStages)], ((g - back) / kHeadStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ========================================================
    if (lane == 0) {
      uint32_t g = 0, n_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++n_tile) {
        const uint32_t acc = n_tile & 1;
        if (n_tile >= 2) ok = wait(HB_ACC_EMPTY + acc, ((n_tile >> 1) - 1) & 1, 200);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < kblocks && ok; ++kb, ++g) {
          const int st = g % kHeadStages;
          ok = wait(HB_FULL + st, (g / kHeadStages) & 1, 210);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = umma_desc_sw128(base + st * kHeadStageBytes, 16, 1024);
          const uint64_t b_desc = umma_desc_sw128(base + st * kHeadStageBytes + kHeadABytes, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < kHeadBK / 16; ++ks)
            umma_bf16_ss(tmem + acc * kHeadBN, a_desc + ((ks * 32) >> 4), b_desc + ((ks * 32) >> 4), IDESC,
                         (kb > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&bars[HB_EMPTY + st]);                  // the stage is free once these products have read it
        }
        if (ok) umma_commit(&bars[HB_ACC_FULL + acc]);
      }
    }
    __syncwarp();
  } else {
    // ============================ epilogue: one thread per row =========================================
    const int quad = warp & 3;                                // my 32 lanes of tensor memory
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    bool ok = true;
    uint32_t n_tile = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++n_tile) {
      const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
      const uint32_t acc = n_tile & 1;
      ok = wait(HB_ACC_FULL + acc, (n_tile >> 1) & 1, 300);
      if (!ok) break;
      tc_fence_after();
      const int col0 = nt * kHeadBN;
      uint32_t best_key = 0, best_col = 0;
      bool have = false;
#pragma unroll 1
      for (int c = 0; c < kHeadBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + acc * kHeadBN + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = col0 + c * 32 + i;
          const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[i]))));
          const uint32_t key = head_sort_key(bits);
          if (col < p.vocab && (!have || key > best_key)) { best_key = key; best_col = static_cast<uint32_t>(col); have = true; }
        }
      }
      if (lane == 0) {                                        // the wait above is warp-wide: the accumulator is read out
        tc_fence_before();
        mbar_arrive(&bars[HB_ACC_EMPTY + acc]);
      }
      const int row = mt * kHeadBM + row_in_tile;
      if (row < p.rows && have)
        atomicMax(p.best + row, (static_cast<unsigned long long>(best_key) << 32) | (0xffffffffu - best_col));
    }
  }

  // ---- the last CTA to get here writes the tokens and clears the scratch -----------------------------
  __threadfence();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
  if (tid == 0) is_last_s = (atomicAdd(p.done, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (is_last_s) {
    __threadfence();
    for (int r = tid; r < p.rows; r += kHeadThreads) {
      const unsigned long long w = *reinterpret_cast<volatile unsigned long long*>(p.best + r);
      const int64_t token = static_cast<int64_t>(0xffffffffu - static_cast<uint32_t>(w & 0xffffffffu));
      p.out[r] = w != 0ull ? token : 0;
      if (p.scatter_table != nullptr) p.scatter_table[p.scatter_index[r]] = w != 0ull ? token : 0;
      p.best[r] = 0ull;
    }
    if (tid == 0) *p.done = 0u;
  }
}

}  // namespace mvb

extern "C" size_t mvb_lm_head_argmax_scratch_bytes(int max_rows) {
  if (max_rows <= 0) return 0;
  return (static_cast<size_t>(max_rows) + 1) * sizeof(unsigned long long);
}

extern "C" int mvb_lm_head_argmax(const void* hidden_states, int64_t x_row_stride, const void* weight,
                                  int64_t w_row_stride, int num_rows, int hidden, int vocab, int64_t* out,
                                  int64_t* scatter_table, const int32_t* scatter_index, void* scratch,
                                  size_t scratch_bytes, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (!hidden_states || !weight || !out || !scratch || num_rows < 0 || hidden <= 0 || vocab <= 0) return kInvalidArgument;
  if ((scatter_table == nullptr) != (scatter_index == nullptr)) return kInvalidArgument;
  if (hidden % kHeadBK != 0) return kUnsupportedShape;
  if (scratch_bytes < mvb_lm_head_argmax_scratch_bytes(num_rows) || !is_aligned(scratch, 8)) return kInvalidArgument;
  if (num_rows == 0) return kOk;
  CUtensorMap xm, wm;
  int rc = make_kv_tensor_map(&xm, hidden_states, num_rows, hidden / kHeadBK, kHeadBK, x_row_stride, kHeadBM);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&wm, weight, vocab, hidden / kHeadBK, kHeadBK, w_row_stride, kHeadBN);
  if (rc != kOk) return rc;
  HeadParams p;
  p.rows = num_rows; p.vocab = vocab; p.hidden = hidden;
  p.m_tiles = (num_rows + kHeadBM - 1) / kHeadBM;
  p.n_tiles = (vocab + kHeadBN - 1) / kHeadBN;
  p.done = static_cast<unsigned int*>(scratch);                // word 0: CTAs finished; then one word per row
  p.best = static_cast<unsigned long long*>(scratch) + 1;
  p.out = out; p.scatter_table = scatter_table; p.scatter_index = scatter_index;
  p.dev_status = dev_status;
  rc = opt_in_dynamic_smem<HeadParams>(reinterpret_cast<const void*>(&lm_head_argmax_kernel), kHeadSmem);
  if (rc != kOk) return rc;
  int grid = sm_count();
  const int tiles = p.m_tiles * p.n_tiles;
  if (grid > tiles) grid = tiles;
  lm_head_argmax_kernel<<<grid, kHeadThreads, kHeadSmem, static_cast<cudaStream_t>(stream)>>>(xm, wm, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}
