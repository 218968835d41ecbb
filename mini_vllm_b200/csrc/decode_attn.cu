// Split-context paged decode attention for sm_100a (HBM-bound).
//
// Work unit: a "CTA tile" of CT tokens of one sequence, all KV heads of a head group.  A
// one-CTA plan kernel (once per step; every layer reuses it) prefix-sums the tile counts and
// hands each of the P persistent CTAs a contiguous range of tiles, so the grid never depends on
// data (CUDA-graph capturable).  Two ways of cutting the tile sequence are weighed per step:
//   even     every CTA gets the same number of tiles (balanced to within one tile whatever the
//            ragged lengths are); a sequence is split wherever a CTA boundary falls inside it and
//            its parts are merged through global memory (see below);
//   aligned  every boundary is moved to the nearest sequence boundary, so no sequence is split and
//            nothing is merged.  Taken when its most loaded CTA has at most a few tiles more than
//            the even cut gives everyone - the price of one merge - which is the case for many
//            short contexts (a sliding-window layer, a batch of young requests).
//
// Inside a CTA every warp owns one KV head (and one 16-token sub-tile when there are more
// warps than heads) and runs its own TMA -> shared-memory ring: the lane-0 thread issues
// 128-byte-swizzled bulk tensor loads of K and V rows gathered through the block table, the
// warp waits on the stage's mbarrier, and then
//     S^T[16 tok x 8 heads] = K[16 x D] . Q^T      (mma.sync m16n8k16, A = K via ldmatrix)
//     online softmax down the token axis            (quad shuffles xor 4/8/16)
//     O^T[D x 8 heads]     += V^T[D x 16] . P^T     (A = V via ldmatrix.trans, B = P^T via movmatrix)
// so the G query heads of a GQA group share each loaded K/V tile and the accumulators cost
// D/4 registers per thread.  The arithmetic is a few percent of the issue slots; the kernel is
// bound by the K/V stream: algorithmic bytes = sum_b visible_tokens(b) * 2 * Hkv * D * 2.
//
// A segment (the part of a sequence inside one CTA's range) that covers the whole sequence is
// normalised and written straight to the output; otherwise the CTA writes a partial
// (normalised O in fp32 + log2-sum-exp), bumps the sequence's arrival counter, and the CTA that
// arrives last merges the partials (the combine pass) and re-arms the counter.  Nothing ever
// waits on another CTA, so the launch cannot hang and needs no co-residency.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"
#include "scan.cuh"

namespace mvb {

constexpr int kMaxCtas = 160;          // workspace is sized for this many persistent CTAs
constexpr int kPlanThreads = 256;
constexpr int kMinTilesPerCta = 2;
constexpr int kMaxPartsPerSeq = 32;   // target bound on the partials one sequence is split into
constexpr int kMergeTiles = 4;        // what a partial + arrival + merge costs a CTA, in 64 KB tiles of streaming

struct DecodeHeader {                  // first 32 bytes of the workspace (device memory)
  int32_t total_tiles, per_cta, num_ctas, cta_tokens, num_seqs, window_left, aligned, pad1;
};

// What a CTA needs to start streaming, written by the plan kernel so that the attention kernel
// begins with ONE 32-byte load instead of a chain of dependent ones.
struct alignas(32) CtaDesc {
  int32_t t0, t1;             // this CTA's tile range [t0, t1) (t0 >= t1: no work)
  int32_t b;                  // sequence holding tile t0
  int32_t tp0, tp1;           // that sequence's tile range
  int32_t n;                  // its context length
  int32_t per;                // tiles per CTA
  int32_t blk0;               // block id holding tile t0 (-1: read it from the block table)
};

struct DecodeLayout {                  // byte offsets inside the workspace
  size_t descs, lse, o, tile_prefix, total;       // arrival counters follow tile_prefix[num_seqs + 1]
};

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static DecodeLayout decode_layout(int max_seqs, int hq, int d) {
  DecodeLayout l;
  l.descs = sizeof(DecodeHeader);
  l.lse = align_up(l.descs + sizeof(CtaDesc) * kMaxCtas, 256);
  l.o = align_up(l.lse + sizeof(float) * kMaxCtas * 2 * hq, 256);
  l.tile_prefix = align_up(l.o + sizeof(float) * kMaxCtas * 2 * static_cast<size_t>(hq) * d, 256);
  l.total = align_up(l.tile_prefix + sizeof(int32_t) * (static_cast<size_t>(max_seqs) + 1) +
                         sizeof(int32_t) * static_cast<size_t>(max_seqs) * hq, 256);
  return l;
}

template <int D, int HPC>
struct DecodeCfg {
  static constexpr int NW = (D == 128) ? 8 : 4;       // warps per CTA
  static constexpr int TS = NW / HPC;                 // 16-token sub-tiles per CTA tile
  static constexpr int CT = TS * 16;                  // tokens per CTA tile
  static constexpr int NSTAGES = 3;
  static constexpr int HALVES = D / 64;               // 64-element (128-byte) column halves
  static constexpr int TILE_BYTES = 16 * D * 2;       // K (or V) rows of one sub-tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int FIN_STRIDE = D + 4;            // floats per (warp, head): O[D], m, l
  static_assert(NW % HPC == 0, "warps must divide evenly over the heads of a CTA");
};

static int cta_tokens_for(int hkv, int d) {
  const int nw = d == 128 ? 8 : 4;
  const int hpc = hkv < nw ? hkv : nw;
  return (nw / hpc) * 16;
}

// ---- plan -------------------------------------------------------------------------------------
__device__ __forceinline__ int visible_start(int n, int window_left) {
  return window_left >= 0 ? max(0, n - 1 - window_left) : 0;
}

__global__ void __launch_bounds__(kPlanThreads) decode_plan_kernel(const int32_t* __restrict__ cache_seqlens,
                                                                   int num_seqs, int window_left, int cta_tokens,
                                                                   int num_ctas, int num_counters,
                                                                   const int32_t* __restrict__ block_table,
                                                                   int64_t table_stride, int block_size,
                                                                   DecodeHeader* hdr, CtaDesc* descs,
                                                                   int32_t* tile_prefix) {
  __shared__ int max_tiles_s, max_load_s;
  if (threadIdx.x == 0) { max_tiles_s = 0; max_load_s = 0; }
  for (int i = threadIdx.x; i < num_counters; i += kPlanThreads) tile_prefix[num_seqs + 1 + i] = 0;
  __syncthreads();
  block_exclusive_scan<kPlanThreads>(
      [&](int b) {
        const int n = cache_seqlens[b];
        if (n <= 0) return 0;
        const int start_al = visible_start(n, window_left) / cta_tokens * cta_tokens;
        const int tiles = (n - start_al + cta_tokens - 1) / cta_tokens;
        atomicMax(&max_tiles_s, tiles);
        return tiles;
      },
      num_seqs, tile_prefix);
  const int total = tile_prefix[num_seqs];
  int per = (total + num_ctas - 1) / num_ctas;
  per = per < kMinTilesPerCta ? kMinTilesPerCta : per;
  // one CTA merges all partials of a sequence: keep that bounded (a few-sequence batch would
  // otherwise be cut into a hundred slivers whose merge costs more than the streaming)
  const int per_for_merge = (max_tiles_s + kMaxPartsPerSeq - 1) / kMaxPartsPerSeq;
  per = per < per_for_merge ? per_for_merge : per;
  auto seq_of_tile = [&](int t) -> int {   // last b with tile_prefix[b] <= t (the sequence holding tile t < total)
    int lo = 0, hi = num_seqs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_prefix[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
  };
  // the aligned cut: boundary c sits on the sequence boundary nearest to c * total / num_ctas
  auto aligned_start = [&](int c) -> int {
    if (c <= 0 || total == 0) return 0;
    if (c >= num_ctas) return total;
    const int ideal = static_cast<int>(static_cast<int64_t>(c) * total / num_ctas);
    const int b = seq_of_tile(ideal);
    const int below = tile_prefix[b], above = tile_prefix[b + 1];
    return ideal - below <= above - ideal ? below : above;
  };
  for (int c = threadIdx.x; c < num_ctas; c += kPlanThreads)
    atomicMax(&max_load_s, aligned_start(c + 1) - aligned_start(c));
  __syncthreads();
  const bool aligned = total > 0 && max_load_s <= per + kMergeTiles;
  if (threadIdx.x == 0) {
    hdr->total_tiles = total; hdr->per_cta = per; hdr->num_ctas = num_ctas; hdr->cta_tokens = cta_tokens;
    hdr->num_seqs = num_seqs; hdr->window_left = window_left; hdr->aligned = aligned ? 1 : 0; hdr->pad1 = 0;
  }
  for (int c = threadIdx.x; c < num_ctas; c += kPlanThreads) {
    const int64_t even0 = static_cast<int64_t>(c) * per;
    const int64_t t = aligned ? aligned_start(c) : even0;
    CtaDesc d;
    d.t0 = t < total ? static_cast<int32_t>(t) : total;
    d.t1 = aligned ? aligned_start(c + 1) : (even0 + per < total ? static_cast<int32_t>(even0 + per) : total);
    d.b = num_seqs; d.tp0 = d.tp1 = d.n = 0; d.per = per; d.blk0 = -1;
    if (d.t0 < d.t1) {
      const int lo = seq_of_tile(d.t0);
      d.b = lo; d.tp0 = tile_prefix[lo]; d.tp1 = tile_prefix[lo + 1]; d.n = cache_seqlens[lo];
      if (block_table != nullptr) {      // spare the attention kernel one dependent load before its first TMA
        const int start_al = visible_start(d.n, window_left) / cta_tokens * cta_tokens;
        const int token0 = start_al + (static_cast<int>(t) - d.tp0) * cta_tokens;
        d.blk0 = block_table[lo * table_stride + token0 / block_size];
      }
    }
    descs[c] = d;
  }
}

// ---- main kernel ------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  __nv_bfloat16* out;
  int64_t out_stride;
  const int32_t* cache_seqlens;
  const int32_t* block_table;
  int64_t table_stride;
  int table_width;
  int num_seqs, hq, group, block_size;
  int64_t num_blocks;
  float scale_log2;
  int window_left;
  const DecodeHeader* hdr;
  const CtaDesc* descs;
  const int32_t* tile_prefix;
  float* part_lse;
  float* part_o;
  int32_t* arrivals;            // [num_seqs * gridDim.y], zero between launches
  int* dev_status;
};

struct SeqView {
  int b, tp0, tp1, n, start, start_al;
};

template <int CT>
__device__ __forceinline__ void load_seq(SeqView& s, int b, const DecodeParams& p) {
  s.b = b;
  s.tp0 = p.tile_prefix[b];
  s.tp1 = p.tile_prefix[b + 1];
  s.n = p.cache_seqlens[b];
  s.start = visible_start(s.n, p.window_left);
  s.start_al = s.start / CT * CT;
}

template <int D, int HPC>
__global__ void __launch_bounds__(DecodeCfg<D, HPC>::NW * 32, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                   const DecodeParams p) {
  using C = DecodeCfg<D, HPC>;
  constexpr int NW = C::NW, CT = C::CT, NST = C::NSTAGES;
  constexpr uint32_t FULL = 0xffffffffu;
  extern __shared__ uint8_t smem_raw[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head_local = warp % HPC, sub = warp / HPC;
  const int kvh = blockIdx.y * HPC + head_local;
  const int G = p.group;
  const int c = blockIdx.x;
  CtaDesc desc;
  {
    const int4* dp = reinterpret_cast<const int4*>(p.descs + c);
    const int4 lo = __ldg(dp), hi = __ldg(dp + 1);
    desc.t0 = lo.x; desc.t1 = lo.y; desc.b = lo.z; desc.tp0 = lo.w;
    desc.tp1 = hi.x; desc.n = hi.y; desc.per = hi.z; desc.blk0 = hi.w;
  }
  const int per = desc.per, t0 = desc.t0, t1 = desc.t1;
  // rows with an empty context (graph padding) produce zeros; spread over the CTAs, and done by
  // idle CTAs first so it stays off the path of the ones that stream
  auto zero_empty_rows = [&]() {
    for (int b = c; b < p.num_seqs; b += gridDim.x) {
      if (p.cache_seqlens[b] <= 0) {
        __nv_bfloat16* row = p.out + b * p.out_stride + static_cast<int64_t>(blockIdx.y) * HPC * G * D;
        for (int e = threadIdx.x; e < HPC * G * D; e += NW * 32) row[e] = __float2bfloat16_rn(0.f);
      }
    }
  };
  if (t0 >= t1) {                                            // CTA-uniform: nothing to stream
    zero_empty_rows();
    return;
  }

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t my_stages = base + warp * (NST * C::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + NW * NST * C::STAGE_BYTES) + warp * NST;
  float* fin = reinterpret_cast<float*>(base_ptr + NW * NST * C::STAGE_BYTES + NW * NST * sizeof(uint64_t));

  if (lane == 0) {
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
#pragma unroll
    for (int s = 0; s < NST; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncwarp();                                              // a warp's barriers are armed and waited on by itself only

  // ---- producer side: the same tile walk as the consumer, NST-1 tiles ahead --------------------
  auto seq_from_desc = [&](SeqView& v) {
    v.b = desc.b; v.tp0 = desc.tp0; v.tp1 = desc.tp1; v.n = desc.n;
    v.start = visible_start(v.n, p.window_left);
    v.start_al = v.start / CT * CT;
  };
  SeqView fs;
  seq_from_desc(fs);
  // lane i caches the block id of table column blk_base + i (blk_n valid lanes); seeded from the plan
  int ft = t0, nfetch = 0, blk_base = -1, blk_reg = -1, blk_n = 0;
  if (desc.blk0 >= 0) {
    blk_base = (fs.start_al + (t0 - fs.tp0) * CT) / p.block_size;
    blk_reg = desc.blk0;
    blk_n = 1;
  }
  auto fetch_next = [&]() -> bool {
    while (true) {
      if (ft >= t1) return false;
      while (ft >= fs.tp1 && fs.b + 1 < p.num_seqs) { load_seq<CT>(fs, fs.b + 1, p); blk_base = -1; blk_n = 0; }
      const int token0 = fs.start_al + (ft - fs.tp0) * CT + sub * 16;
      ++ft;
      if (token0 >= fs.n || token0 + 16 <= fs.start) continue;
      const int bi = token0 / p.block_size;
      if (blk_base < 0 || bi < blk_base || bi >= blk_base + blk_n) {
        blk_base = bi;
        blk_n = 32;
        const int col = bi + lane;
        blk_reg = col < p.table_width ? p.block_table[fs.b * p.table_stride + col] : -1;
      }
      const int blk = __shfl_sync(FULL, blk_reg, bi - blk_base);
      int slot0 = -16;                                       // out of range -> TMA zero fill
      if (blk >= 0 && blk < p.num_blocks) slot0 = blk * p.block_size + (token0 - bi * p.block_size);
      else if (lane == 0) report(p.dev_status, kDevBadBlock, fs.b);
      if (lane == 0) {
        const int st = nfetch % NST;
        const uint32_t kdst = my_stages + st * C::STAGE_BYTES;
        mbar_arrive_expect_tx(&bars[st], C::STAGE_BYTES);
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) {
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(kdst + h * 2048), "l"(reinterpret_cast<uint64_t>(&k_map)), "r"(smem_u32(&bars[st])),
                "r"(h * 64), "r"(kvh), "r"(slot0) : "memory");
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(kdst + C::TILE_BYTES + h * 2048), "l"(reinterpret_cast<uint64_t>(&v_map)),
                "r"(smem_u32(&bars[st])), "r"(h * 64), "r"(kvh), "r"(slot0) : "memory");
        }
      }
      ++nfetch;
      return true;
    }
  };
#pragma unroll
  for (int i = 0; i < NST - 1; ++i) fetch_next();

  // ---- consumer side ------------------------------------------------------------------------------
  SeqView cs;
  seq_from_desc(cs);
  const int first_b = cs.b;
  int t = t0, ncomp = 0;
  bool dead = false;

  while (t < t1) {
    while (t >= cs.tp1 && cs.b + 1 < p.num_seqs) load_seq<CT>(cs, cs.b + 1, p);
    const int seg_end = min(t1, cs.tp1);
    const bool whole = (t == cs.tp0) && (seg_end == cs.tp1);
    const int b = cs.b;

    // Q^T as the B operand: lane holds head (lane/4) of the group, dims ks*16 + (lane%4)*2 + {0,1,8,9}
    uint32_t qf[D / 16][2];
    {
      const int g = lane >> 2;
      const __nv_bfloat16* qrow = p.q + b * p.q_stride + (static_cast<int64_t>(kvh) * G + g) * D + (lane & 3) * 2;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16) : 0u;
        qf[ks][1] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8) : 0u;
      }
    }
    float o[D / 16][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) { o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    for (; t < seg_end; ++t) {
      const int token0 = cs.start_al + (t - cs.tp0) * CT + sub * 16;
      if (token0 >= cs.n || token0 + 16 <= cs.start) continue;
      if (dead) continue;
      fetch_next();
      const int st = ncomp % NST;
      const uint32_t parity = (ncomp / NST) & 1;
      const bool ok = mbar_wait(&bars[st], parity);
      if (!__all_sync(FULL, ok)) {
        if (lane == 0) report(p.dev_status, kDevWaitTimeout, ncomp);
        dead = true;
        continue;
      }
      ++ncomp;
      const uint32_t kbase = my_stages + st * C::STAGE_BYTES;
      const uint32_t vbase = kbase + C::TILE_BYTES;

      // rows past the end of the sequence may hold anything (even NaN): zero them in V
      const int valid = cs.n - token0;
      if (valid < 16) {
        const int chunks = (16 - valid) * C::HALVES * 8;
        for (int i = lane; i < chunks; i += 32) {
          const int r = valid + i / (C::HALVES * 8), rem = i % (C::HALVES * 8);
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(vbase + (rem >> 3) * 2048 + r * 128 + (rem & 7) * 16),
                       "r"(0) : "memory");
        }
        __syncwarp();
      }

      // S^T = K . Q^T
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const uint32_t rbase = kbase + row * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const int chunk = ks * 2 + (lane >> 4);
          uint32_t a[4];
          ldmatrix_x4(a, rbase + (chunk >> 3) * 2048 + (((chunk & 7) ^ (row & 7)) << 4));
          if (ks & 1) mma_bf16_16816(s1, a, qf[ks][0], qf[ks][1]);
          else mma_bf16_16816(s0, a, qf[ks][0], qf[ks][1]);
        }
      }
      const int j0 = token0 + (lane >> 2), j1 = j0 + 8;
      const bool v0 = j0 < cs.n && j0 >= cs.start, v1 = j1 < cs.n && j1 >= cs.start;
      const float x0 = v0 ? (s0[0] + s1[0]) * p.scale_log2 : -INFINITY;
      const float x1 = v0 ? (s0[1] + s1[1]) * p.scale_log2 : -INFINITY;
      const float x2 = v1 ? (s0[2] + s1[2]) * p.scale_log2 : -INFINITY;
      const float x3 = v1 ? (s0[3] + s1[3]) * p.scale_log2 : -INFINITY;
      float ta = fmaxf(x0, x2), tb = fmaxf(x1, x3);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        ta = fmaxf(ta, __shfl_xor_sync(FULL, ta, off));
        tb = fmaxf(tb, __shfl_xor_sync(FULL, tb, off));
      }
      const float na = fmaxf(m_a, ta), nb = fmaxf(m_b, tb);
      const float sa = na == -INFINITY ? 0.f : na, sb = nb == -INFINITY ? 0.f : nb;
      const float alpha_a = fast_exp2(m_a - sa), alpha_b = fast_exp2(m_b - sb);
      const float p0 = fast_exp2(x0 - sa), p1 = fast_exp2(x1 - sb), p2 = fast_exp2(x2 - sa), p3 = fast_exp2(x3 - sb);
      l_a = l_a * alpha_a + p0 + p2;
      l_b = l_b * alpha_b + p1 + p3;
      m_a = na; m_b = nb;
      const uint32_t pb0 = movmatrix_trans(pack_bf16(p0, p1));
      const uint32_t pb1 = movmatrix_trans(pack_bf16(p2, p3));

      // O^T = O^T * alpha + V^T . P^T
      {
        const int mi = lane >> 3;
        const int tok = (lane & 7) + (mi >> 1) * 8;
        const uint32_t rbase = vbase + tok * 128;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
          const int chunk = mt * 2 + (mi & 1);
          uint32_t a[4];
          ldmatrix_x4_trans(a, rbase + (chunk >> 3) * 2048 + (((chunk & 7) ^ (tok & 7)) << 4));
          o[mt][0] *= alpha_a; o[mt][1] *= alpha_b; o[mt][2] *= alpha_a; o[mt][3] *= alpha_b;
          mma_bf16_16816(o[mt], a, pb0, pb1);
        }
      }
      __syncwarp();
    }
    // ---- end of segment: merge the warps that share a head, then write output or partial --------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l_a += __shfl_xor_sync(FULL, l_a, off);
      l_b += __shfl_xor_sync(FULL, l_b, off);
    }
    {
      const int ha = (lane & 3) * 2, r = lane >> 2;
      float* fa = fin + (warp * G + ha) * C::FIN_STRIDE;
      float* fb = fa + C::FIN_STRIDE;
      if (ha < G) {
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) { fa[mt * 16 + r] = o[mt][0]; fa[mt * 16 + r + 8] = o[mt][2]; }
        if (r == 0) { fa[D] = m_a; fa[D + 1] = l_a; }
      }
      if (ha + 1 < G) {
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) { fb[mt * 16 + r] = o[mt][1]; fb[mt * 16 + r + 8] = o[mt][3]; }
        if (r == 0) { fb[D] = m_b; fb[D + 1] = l_b; }
      }
    }
    __syncthreads();
    const float* __restrict__ plse = p.part_lse;
    const float* __restrict__ po = p.part_o;
    float* __restrict__ plse_w = p.part_lse;
    float* __restrict__ po_w = p.part_o;
    __nv_bfloat16* __restrict__ outp = p.out;
    const int heads = HPC * G;                               // query heads of this CTA
    const int items = heads * D / 4;                         // 4-dim groups to produce
    {
      const int slot = (b == first_b) ? 0 : 1;
      for (int it = threadIdx.x; it < items; it += NW * 32) {
        const int h = (it * 4) / D, dim = (it * 4) % D;      // h = hl * G + g
        const int hl = h / G, g = h - hl * G;
        float M = -INFINITY;
#pragma unroll
        for (int sb = 0; sb < C::TS; ++sb) M = fmaxf(M, fin[((sb * HPC + hl) * G + g) * C::FIN_STRIDE + D]);
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int sb = 0; sb < C::TS; ++sb) {
          const float* f = fin + ((sb * HPC + hl) * G + g) * C::FIN_STRIDE;
          const float w = f[D] == -INFINITY ? 0.f : fast_exp2(f[D] - M);
          const float4 v = *reinterpret_cast<const float4*>(f + dim);
          L += f[D + 1] * w;
          acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        const int qh = blockIdx.y * heads + h;
        if (whole) {
          uint2 w2;
          w2.x = pack_bf16(acc.x, acc.y); w2.y = pack_bf16(acc.z, acc.w);
          *reinterpret_cast<uint2*>(outp + b * p.out_stride + static_cast<int64_t>(qh) * D + dim) = w2;
        } else {
          const int64_t pi = (static_cast<int64_t>(c) * 2 + slot) * p.hq + qh;
          *reinterpret_cast<float4*>(po_w + pi * D + dim) = acc;
          if (dim == 0) plse_w[pi] = L > 0.f ? M + log2f(L) : -INFINITY;
        }
      }
    }
    if (!whole) {
      // combine pass without waiting: publish the partial, count the arrival; whoever arrives last
      // finds every partial of this sequence in memory and merges them
      __shared__ int is_last;
      const int c1 = cs.tp0 / per, c2 = (cs.tp1 - 1) / per;
      // the CTA barrier orders every thread's partial stores before thread 0's release; the last
      // arriver's acquire plus its CTA barrier order them before every merging thread's loads
      __syncthreads();
      if (threadIdx.x == 0) {
        int32_t* cnt = p.arrivals + static_cast<int64_t>(b) * gridDim.y + blockIdx.y;
        int prev;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(cnt) : "memory");
        is_last = (prev == c2 - c1);
        if (is_last) *cnt = 0;                               // re-arm for the next launch
      }
      __syncthreads();
      if (is_last) {
        constexpr int HEADS = HPC * 8;                       // upper bound of HPC * G
        constexpr int PC = 32;                               // partials weighted per pass
        constexpr int MAX_ITEMS = (HEADS * D / 4 + NW * 32 - 1) / (NW * 32);
        int* m_enc = reinterpret_cast<int*>(fin);            // per-head max of the partial LSEs, order-encoded
        float* w_s = fin + HEADS;                            // [PC][heads] weights of the current pass
        const int nparts = c2 - c1 + 1;
        const bool first_is_head = (cs.tp0 % per) == 0;      // does CTA c1's range start at this sequence?
        auto part_index = [&](int cc, int qh) -> int64_t {
          const int sl = (cc > c1 || first_is_head) ? 0 : 1;
          return (static_cast<int64_t>(cc) * 2 + sl) * p.hq + qh;
        };
        if (threadIdx.x < HEADS) m_enc[threadIdx.x] = INT_MIN;
        __syncthreads();
        for (int i = threadIdx.x; i < nparts * heads; i += NW * 32) {
          const int h = i % heads;
          const int bits = __float_as_int(__ldcg(plse + part_index(c1 + i / heads, blockIdx.y * heads + h)));
          atomicMax(&m_enc[h], bits >= 0 ? bits : bits ^ 0x7fffffff);
        }
        __syncthreads();
        float4 acc[MAX_ITEMS];
        float wsum[MAX_ITEMS];
#pragma unroll
        for (int k = 0; k < MAX_ITEMS; ++k) { acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); wsum[k] = 0.f; }
        for (int p0 = 0; p0 < nparts; p0 += PC) {
          const int pn = min(PC, nparts - p0);
          for (int i = threadIdx.x; i < pn * heads; i += NW * 32) {
            const int h = i % heads;
            const int enc = m_enc[h];
            const float M = __int_as_float(enc >= 0 ? enc : enc ^ 0x7fffffff);
            const float lse = __ldcg(plse + part_index(c1 + p0 + i / heads, blockIdx.y * heads + h));
            w_s[i] = lse == -INFINITY ? 0.f : fast_exp2(lse - M);
          }
          __syncthreads();
#pragma unroll
          for (int k = 0; k < MAX_ITEMS; ++k) {
            const int it = threadIdx.x + k * NW * 32;
            if (it < items) {
              const int h = (it * 4) / D, dim = (it * 4) % D, qh = blockIdx.y * heads + h;
#pragma unroll 8
              for (int j = 0; j < pn; ++j) {                 // independent 16-byte loads: they pipeline
                const float w = w_s[j * heads + h];
                const float4 v = __ldcg(reinterpret_cast<const float4*>(po + part_index(c1 + p0 + j, qh) * D + dim));
                acc[k].x = fmaf(w, v.x, acc[k].x); acc[k].y = fmaf(w, v.y, acc[k].y);
                acc[k].z = fmaf(w, v.z, acc[k].z); acc[k].w = fmaf(w, v.w, acc[k].w);
                wsum[k] += w;
              }
            }
          }
          __syncthreads();
        }
#pragma unroll
        for (int k = 0; k < MAX_ITEMS; ++k) {
          const int it = threadIdx.x + k * NW * 32;
          if (it < items) {
            const int h = (it * 4) / D, dim = (it * 4) % D, qh = blockIdx.y * heads + h;
            const float inv = wsum[k] > 0.f ? 1.f / wsum[k] : 0.f;
            uint2 w2;
            w2.x = pack_bf16(acc[k].x * inv, acc[k].y * inv); w2.y = pack_bf16(acc[k].z * inv, acc[k].w * inv);
            *reinterpret_cast<uint2*>(outp + b * p.out_stride + static_cast<int64_t>(qh) * D + dim) = w2;
          }
        }
      }
    }
    __syncthreads();
  }
  zero_empty_rows();

  // a wait that gave up may leave copies in flight: give them a bounded chance to land
  if (dead) {
    for (int i = ncomp; i < nfetch; ++i) mbar_wait(&bars[i % NST], (i / NST) & 1, 1u << 16);
  }
}

template <int D, int HPC>
static int launch_decode(const CUtensorMap& km, const CUtensorMap& vm, const DecodeParams& p, int hkv, int num_ctas,
                         cudaStream_t stream) {
  using C = DecodeCfg<D, HPC>;
  const size_t smem = 1024 + static_cast<size_t>(C::NW) * C::NSTAGES * C::STAGE_BYTES +
                      C::NW * C::NSTAGES * sizeof(uint64_t) +
                      static_cast<size_t>(C::NW) * p.group * C::FIN_STRIDE * sizeof(float);
  if (smem + 64 > 227 * 1024) return kUnsupportedShape;       // static shared memory counts too
  const int rc = opt_in_dynamic_smem<C>(reinterpret_cast<const void*>(&decode_attn_kernel<D, HPC>), smem);
  if (rc != kOk) return rc;
  dim3 grid(num_ctas, hkv / HPC);
  decode_attn_kernel<D, HPC><<<grid, C::NW * 32, smem, stream>>>(km, vm, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace mvb

extern "C" size_t mvb_decode_workspace_bytes(int max_seqs, int num_q_heads, int head_dim) {
  if (max_seqs <= 0 || num_q_heads <= 0 || head_dim <= 0) return 0;
  return mvb::decode_layout(max_seqs, num_q_heads, head_dim).total;
}

static int decode_shape_ok(int hq, int hkv, int d) {
  if (hq <= 0 || hkv <= 0 || hq % hkv != 0) return 0;
  if (d != 128 && d != 256) return 0;
  const int g = hq / hkv;
  if (g > 8) return 0;
  const int nw = d == 128 ? 8 : 4;
  if (hkv < nw) return (hkv == 1 || hkv == 2 || hkv == 4);
  return hkv % nw == 0;
}

// Everything about a decode-attention call that can be rejected before anything is enqueued.
static int decode_check_args(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                             int64_t num_blocks, int block_size, const int32_t* cache_seqlens,
                             const int32_t* block_table, int64_t table_stride, int table_width, int num_seqs,
                             int num_q_heads, int num_kv_heads, int head_dim, const void* out,
                             int64_t out_row_stride) {
  using namespace mvb;
  if (!q || !k_cache || !v_cache || !cache_seqlens || !block_table || !out) return kInvalidArgument;
  if (num_seqs <= 0 || num_blocks <= 0 || block_size <= 0 || table_width <= 0 || table_stride < table_width)
    return kInvalidArgument;
  if (!decode_shape_ok(num_q_heads, num_kv_heads, head_dim)) return kUnsupportedShape;
  if (block_size % 16 != 0) return kUnsupportedShape;
  if (num_blocks * block_size > 0x7fffffffLL) return kUnsupportedShape;
  if ((q_row_stride % 2) || (out_row_stride % 4) || !is_aligned(q, 4) || !is_aligned(out, 8)) return kMisaligned;
  if (!is_aligned(k_cache, 16) || !is_aligned(v_cache, 16)) return kMisaligned;
  return kOk;
}

static int decode_plan_impl(const int32_t* cache_seqlens, const int32_t* block_table, int64_t table_stride,
                            int block_size, int num_seqs, int window_left, int num_q_heads, int num_kv_heads,
                            int head_dim, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mvb;
  if (!cache_seqlens || !workspace || num_seqs <= 0) return kInvalidArgument;
  if (!decode_shape_ok(num_q_heads, num_kv_heads, head_dim)) return kUnsupportedShape;
  const DecodeLayout l = decode_layout(num_seqs, num_q_heads, head_dim);
  if (workspace_bytes < l.total || !is_aligned(workspace, 256)) return kInvalidArgument;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int num_ctas = sm_count();
  if (num_ctas > kMaxCtas) num_ctas = kMaxCtas;
  decode_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      cache_seqlens, num_seqs, window_left, cta_tokens_for(num_kv_heads, head_dim), num_ctas,
      num_seqs * num_q_heads, block_table, table_stride, block_size, reinterpret_cast<DecodeHeader*>(ws),
      reinterpret_cast<CtaDesc*>(ws + l.descs), reinterpret_cast<int32_t*>(ws + l.tile_prefix));
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

extern "C" int mvb_decode_plan(const int32_t* cache_seqlens, int num_seqs, int window_left, int num_q_heads,
                               int num_kv_heads, int head_dim, void* workspace, size_t workspace_bytes,
                               void* stream) {
  return decode_plan_impl(cache_seqlens, nullptr, 0, 0, num_seqs, window_left, num_q_heads, num_kv_heads, head_dim,
                          workspace, workspace_bytes, stream);
}

extern "C" int mvb_decode_plan_with_table(const int32_t* cache_seqlens, const int32_t* block_table,
                                          int64_t table_stride, int block_size, int num_seqs, int window_left,
                                          int num_q_heads, int num_kv_heads, int head_dim, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  if (!block_table || block_size <= 0 || table_stride <= 0) return mvb::kInvalidArgument;
  return decode_plan_impl(cache_seqlens, block_table, table_stride, block_size, num_seqs, window_left, num_q_heads,
                          num_kv_heads, head_dim, workspace, workspace_bytes, stream);
}

extern "C" int mvb_decode_attn(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                               int64_t num_blocks, int block_size, const int32_t* cache_seqlens,
                               const int32_t* block_table, int64_t table_stride, int table_width, int num_seqs,
                               int num_q_heads, int num_kv_heads, int head_dim, float scale, int window_left,
                               void* out, int64_t out_row_stride, void* workspace, size_t workspace_bytes,
                               int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (!workspace) return kInvalidArgument;
  int rc = decode_check_args(q, q_row_stride, k_cache, v_cache, num_blocks, block_size, cache_seqlens, block_table,
                             table_stride, table_width, num_seqs, num_q_heads, num_kv_heads, head_dim, out,
                             out_row_stride);
  if (rc != kOk) return rc;
  const DecodeLayout l = decode_layout(num_seqs, num_q_heads, head_dim);
  if (workspace_bytes < l.total || !is_aligned(workspace, 256)) return kInvalidArgument;

  CUtensorMap km, vm;
  const int64_t rows = num_blocks * block_size;
  rc = make_kv_tensor_map(&km, k_cache, rows, num_kv_heads, head_dim, static_cast<int64_t>(num_kv_heads) * head_dim, 16);
  if (rc != kOk) return rc;
  rc = make_kv_tensor_map(&vm, v_cache, rows, num_kv_heads, head_dim, static_cast<int64_t>(num_kv_heads) * head_dim, 16);
  if (rc != kOk) return rc;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride = q_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_row_stride;
  p.cache_seqlens = cache_seqlens; p.block_table = block_table; p.table_stride = table_stride;
  p.table_width = table_width;
  p.num_seqs = num_seqs; p.hq = num_q_heads; p.group = num_q_heads / num_kv_heads; p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window_left = window_left;
  p.hdr = reinterpret_cast<const DecodeHeader*>(ws);
  p.descs = reinterpret_cast<const CtaDesc*>(ws + l.descs);
  p.tile_prefix = reinterpret_cast<const int32_t*>(ws + l.tile_prefix);
  p.part_lse = reinterpret_cast<float*>(ws + l.lse);
  p.part_o = reinterpret_cast<float*>(ws + l.o);
  p.arrivals = reinterpret_cast<int32_t*>(ws + l.tile_prefix) + num_seqs + 1;
  p.dev_status = dev_status;

  int num_ctas = sm_count();
  if (num_ctas > kMaxCtas) num_ctas = kMaxCtas;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nw = head_dim == 128 ? 8 : 4;
  const int hpc = num_kv_heads < nw ? num_kv_heads : nw;
  rc = kUnsupportedShape;
  if (head_dim == 128) {
    if (hpc == 8) rc = launch_decode<128, 8>(km, vm, p, num_kv_heads, num_ctas, st);
    else if (hpc == 4) rc = launch_decode<128, 4>(km, vm, p, num_kv_heads, num_ctas, st);
    else if (hpc == 2) rc = launch_decode<128, 2>(km, vm, p, num_kv_heads, num_ctas, st);
    else if (hpc == 1) rc = launch_decode<128, 1>(km, vm, p, num_kv_heads, num_ctas, st);
  } else {
    if (hpc == 4) rc = launch_decode<256, 4>(km, vm, p, num_kv_heads, num_ctas, st);
    else if (hpc == 2) rc = launch_decode<256, 2>(km, vm, p, num_kv_heads, num_ctas, st);
    else if (hpc == 1) rc = launch_decode<256, 1>(km, vm, p, num_kv_heads, num_ctas, st);
  }
  return rc;
}

// ---- decode attention without caller-supplied scratch ------------------------------------------------
// Some users of this library cannot hand it a workspace: a serving process whose device memory is
// carved up once at start-up and that has no allocator to ask afterwards, a binding from a runtime
// that only passes through the tensors it already owns, or a latency-critical loop that must never
// reach cudaMalloc (which synchronises the whole device).  For them the plan, the partial results
// and the arrival counters live in the array below, which is part of the loaded module: every GPU
// that loads the library holds these 8 MiB until the process exits.
namespace mvb {

constexpr size_t kStaticScratchBytes = MVB_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

// In host code the array's name only identifies the symbol; the kernels need its address in device
// memory, which differs per device.  Looked up once per device, with that device current.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr_by_device[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kLaunchFailed;
  std::lock_guard<std::mutex> lock(mu);
  if (addr_by_device[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_decode_scratch) != cudaSuccess || ptr == nullptr) return kLaunchFailed;
    addr_by_device[dev] = ptr;
  }
  *out = addr_by_device[dev];
  return kOk;
}

}  // namespace mvb

extern "C" int mvb_decode_attn_static(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                      int64_t num_blocks, int block_size, const int32_t* cache_seqlens,
                                      const int32_t* block_table, int64_t table_stride, int table_width,
                                      int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                      int window_left, void* out, int64_t out_row_stride, int32_t* dev_status,
                                      void* stream) {
  using namespace mvb;
  // every argument is checked before the plan kernel goes out: a negative return means nothing was enqueued
  int rc = decode_check_args(q, q_row_stride, k_cache, v_cache, num_blocks, block_size, cache_seqlens, block_table,
                             table_stride, table_width, num_seqs, num_q_heads, num_kv_heads, head_dim, out,
                             out_row_stride);
  if (rc != kOk) return rc;
  if (decode_layout(num_seqs, num_q_heads, head_dim).total > kStaticScratchBytes) return kScratchTooSmall;
  if (encode_tiled_fn() == nullptr) return kNoDriverEntry;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != kOk) return rc;
  // The plan launch rewrites the descriptors and zeroes the arrival counters, so nothing left in
  // the array by an earlier call is read.
  rc = mvb_decode_plan(cache_seqlens, num_seqs, window_left, num_q_heads, num_kv_heads, head_dim, scratch,
                       kStaticScratchBytes, stream);
  if (rc != kOk) return rc;
  return mvb_decode_attn(q, q_row_stride, k_cache, v_cache, num_blocks, block_size, cache_seqlens, block_table,
                         table_stride, table_width, num_seqs, num_q_heads, num_kv_heads, head_dim, scale,
                         window_left, out, out_row_stride, scratch, kStaticScratchBytes, dev_status, stream);
}
