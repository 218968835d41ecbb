// Fused temperature / top-k / top-p / Gumbel-max sampler (HBM-bound: algorithmic bytes = num_rows * vocab * 2).
// Every row is split over a thread-block cluster of 1-8 CTAs (chosen on the host so that a small batch still
// fills the GPU); the slices' results meet in the cluster's first CTA through distributed shared memory.
//
// Greedy: argmax of float(logit) / T with the lowest index winning ties, which is what
// torch.argmax returns on the same fp32 values.
// Random: keep every entry >= the k-th largest, then the nucleus of probability mass top_p among those, then
// argmax over the kept entries of  logit / T - log(-log(u)),  u from Philox4x32-10 with
// counter (column/4, row, offset_lo, offset_hi), key (seed_lo, seed_hi), word column%4.
//   Usual case (0 < k <= 1024 < vocab): each CTA streams its slice once (DRAM) keeping, per thread, the maxima of
//   two interleaved subsets of what it reads - 1024 sub-maxima per CTA.  Their k-th largest is a value that at
//   least k entries of the slice reach, so every entry of the row's top k that lies in this slice reaches it too.
//   The CTA streams its slice again (L2) and moves the entries that reach it - about k of them - into the first
//   CTA's shared memory.  There, on a list of a few hundred entries at most, each entry counts the entries
//   larger than itself (its rank, for top-k) and their probability mass (for the nucleus): no sort, no
//   histogram, no floating-point atomics.
//   Otherwise (no top-k, k beyond the sub-maxima, NaNs, a list too long to rank pairwise): the first CTA
//   radix-selects with two 256-bin histogram passes (and two more of softmax mass for the nucleus), over the
//   list if it has one, else over the whole row.
#include "common.cuh"
#include "host_util.cuh"
#include "mini_vllm_b200.h"

#include <cooperative_groups.h>

namespace mvb {

constexpr int kSampleThreads = 512;

struct Best {
  float val;
  int idx;
};

// NaN counts as the largest value (torch.argmax does the same); lower index wins ties.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn || bn) return vn && (!bn || i < bi);
  return v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ Best block_argmax(Best b) {
  __shared__ float sv[kSampleThreads / 32];
  __shared__ int si[kSampleThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, b.val, o);
    const int oi = __shfl_xor_sync(0xffffffffu, b.idx, o);
    if (better(ov, oi, b.val, b.idx)) { b.val = ov; b.idx = oi; }
  }
  if (lane == 0) { sv[warp] = b.val; si[warp] = b.idx; }
  __syncthreads();
  if (warp == 0) {
    b.val = lane < kSampleThreads / 32 ? sv[lane] : -INFINITY;
    b.idx = lane < kSampleThreads / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, b.val, o);
      const int oi = __shfl_xor_sync(0xffffffffu, b.idx, o);
      if (better(ov, oi, b.val, b.idx)) { b.val = ov; b.idx = oi; }
    }
  }
  return b;                                                  // valid in warp 0
}

// Calls f(column, raw_bf16_bits) for every column of the row; 128-bit loads when the row allows.
template <class F>
__device__ __forceinline__ void for_each_logit(const uint16_t* row, int vocab, bool vec_ok, F f) {
  if (vec_ok) {
    const int nvec = vocab / 8;
    for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + v * 8);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f(v * 8 + 2 * i, static_cast<uint16_t>(ws[i] & 0xffffu));
        f(v * 8 + 2 * i + 1, static_cast<uint16_t>(ws[i] >> 16));
      }
    }
    for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kSampleThreads) f(c, row[c]);
  } else {
    for (int c = threadIdx.x; c < vocab; c += kSampleThreads) f(c, row[c]);
  }
}

// Calls f(first column, two packed bf16) for every pair of columns; an odd last column comes with -inf
// in the upper half (column == vocab: callers that act on columns must check it).
template <class F>
__device__ __forceinline__ void for_each_word(const uint16_t* row, int vocab, bool vec_ok, F f) {
  if (vec_ok) {
    const int nvec = vocab / 8;
    for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + v * 8);
      f(v * 8, w.x); f(v * 8 + 2, w.y); f(v * 8 + 4, w.z); f(v * 8 + 6, w.w);
    }
    for (int c = nvec * 8 + 2 * threadIdx.x; c < vocab; c += 2 * kSampleThreads) {
      const uint32_t lo = row[c], hi = c + 1 < vocab ? row[c + 1] : 0xff80u;   // -inf pads an odd tail
      f(c, lo | (hi << 16));
    }
  } else {
    for (int c = 2 * threadIdx.x; c < vocab; c += 2 * kSampleThreads) {
      const uint32_t lo = row[c], hi = c + 1 < vocab ? row[c + 1] : 0xff80u;
      f(c, lo | (hi << 16));
    }
  }
}

// The same over one slice of the row (part of parts, split at 16-byte vectors), with four 128-bit loads in
// flight per thread: a CTA streaming its slice is bound by how many bytes it keeps in flight.
template <class F>
__device__ __forceinline__ void for_each_word_slice(const uint16_t* row, int vocab, bool vec_ok, int part, int parts, F f) {
  if (vec_ok) {
    const int nvec = vocab / 8;
    const int v0 = static_cast<int>(static_cast<int64_t>(nvec) * part / parts);
    const int v1 = static_cast<int>(static_cast<int64_t>(nvec) * (part + 1) / parts);
    int v = v0 + threadIdx.x;
    for (; v + 3 * kSampleThreads < v1; v += 4 * kSampleThreads) {
      uint4 w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) w[u] = *reinterpret_cast<const uint4*>(row + (v + u * kSampleThreads) * 8);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = (v + u * kSampleThreads) * 8;
        f(c, w[u].x); f(c + 2, w[u].y); f(c + 4, w[u].z); f(c + 6, w[u].w);
      }
    }
    for (; v < v1; v += kSampleThreads) {
      const uint4 w = *reinterpret_cast<const uint4*>(row + v * 8);
      f(v * 8, w.x); f(v * 8 + 2, w.y); f(v * 8 + 4, w.z); f(v * 8 + 6, w.w);
    }
    if (part == parts - 1) {
      for (int c = nvec * 8 + 2 * threadIdx.x; c < vocab; c += 2 * kSampleThreads) {
        const uint32_t lo = row[c], hi = c + 1 < vocab ? row[c + 1] : 0xff80u;   // -inf pads an odd tail
        f(c, lo | (hi << 16));
      }
    }
  } else {
    const int c0 = static_cast<int>(static_cast<int64_t>(vocab) * part / parts) & ~1;
    const int c1 = part == parts - 1 ? vocab : (static_cast<int>(static_cast<int64_t>(vocab) * (part + 1) / parts) & ~1);
    for (int c = c0 + 2 * threadIdx.x; c < c1; c += 2 * kSampleThreads) {
      const uint32_t lo = row[c], hi = c + 1 < c1 ? row[c + 1] : 0xff80u;
      f(c, lo | (hi << 16));
    }
  }
}

__device__ __forceinline__ float bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// Monotone map bf16 bits -> uint16 (larger float, larger key); -0 and +0 share a key.
__device__ __forceinline__ uint32_t sort_key(uint16_t b) {
  if (b == 0x8000u) b = 0;
  return (b & 0x8000u) ? static_cast<uint32_t>(static_cast<uint16_t>(~b)) : static_cast<uint32_t>(b | 0x8000u);
}

__device__ __forceinline__ uint16_t key_to_bits(uint32_t key) {
  return (key & 0x8000u) ? static_cast<uint16_t>(key ^ 0x8000u) : static_cast<uint16_t>(~key);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct SampleParams {
  const uint16_t* logits;
  int64_t row_stride;
  int vocab;
  const float* temperatures;
  const int32_t* top_k;
  const float* top_p;
  uint64_t seed, offset;
  int64_t* out;
  int64_t* scatter_table;        // optional: table[scatter_index[row]] = token as well
  const int32_t* scatter_index;
};

// Greedy: a cluster of CTAs per row (1, 2, 4 or 8, chosen on the host so that small batches still fill
// the GPU), each over a contiguous slice of the vocabulary with 128-bit loads; the slices' winners
// meet in the first CTA through distributed shared memory.
__global__ void __launch_bounds__(kSampleThreads) sample_greedy_kernel(const SampleParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int parts = static_cast<int>(cluster.num_blocks()), part = static_cast<int>(cluster.block_rank());
  const int r = blockIdx.x / parts;
  __shared__ Best slice_best;
  const uint16_t* row = p.logits + r * p.row_stride;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  const bool scaled = p.temperatures != nullptr;
  const float temp = scaled ? p.temperatures[r] : 1.f;
  Best b{-INFINITY, 0x7fffffff};
  auto consider = [&](int c, uint16_t bits) {
    float x = bits_to_float(bits);
    if (scaled) x = __fdiv_rn(x, temp);
    if (better(x, c, b.val, b.idx)) { b.val = x; b.idx = c; }
  };
  if (vec_ok) {
    const int nvec = p.vocab / 8;
    const int v0 = static_cast<int>(static_cast<int64_t>(nvec) * part / parts);
    const int v1 = static_cast<int>(static_cast<int64_t>(nvec) * (part + 1) / parts);
    auto take = [&](int v, const uint4& w) {
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        consider(v * 8 + 2 * i, static_cast<uint16_t>(ws[i] & 0xffffu));
        consider(v * 8 + 2 * i + 1, static_cast<uint16_t>(ws[i] >> 16));
      }
    };
    bool exact_pass = scaled;
    if (!scaled) {
      // Unscaled rows are compared as packed bf16 pairs: per 32-bit word of the 128-bit load a running
      // maximum of each half and the loop count at which that half last grew (strictly, so the first
      // occurrence stays) - 3 instructions per two logits.  A NaN poisons its running maximum; such a
      // row is then redone by the exact pass below.
      __nv_bfloat162 m[4];
      uint32_t when[4];                                       // two 16-bit loop counts per word, 0xffff = never
#pragma unroll
      for (int i = 0; i < 4; ++i) { m[i] = __floats2bfloat162_rn(-INFINITY, -INFINITY); when[i] = 0xffffffffu; }
      const int vstart = v0 + threadIdx.x;
      uint32_t count2 = 0;                                    // loop count in both halves
#pragma unroll 4
      for (int v = vstart; v < v1; v += kSampleThreads, count2 += 0x00010001u) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + v * 8);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&ws[i]);
          const uint32_t grew = __hgt2_mask(x, m[i]);
          m[i] = __hmax2_nan(m[i], x);
          when[i] = (grew & count2) | (~grew & when[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __low2float(m[i]), hi = __high2float(m[i]);
        if (lo != lo || hi != hi) exact_pass = true;
        const uint32_t wl = when[i] & 0xffffu, wh = when[i] >> 16;
        if (wl != 0xffffu && better(lo, (vstart + static_cast<int>(wl) * kSampleThreads) * 8 + 2 * i, b.val, b.idx)) {
          b.val = lo; b.idx = (vstart + static_cast<int>(wl) * kSampleThreads) * 8 + 2 * i;
        }
        if (wh != 0xffffu && better(hi, (vstart + static_cast<int>(wh) * kSampleThreads) * 8 + 2 * i + 1, b.val, b.idx)) {
          b.val = hi; b.idx = (vstart + static_cast<int>(wh) * kSampleThreads) * 8 + 2 * i + 1;
        }
      }
      exact_pass = __syncthreads_or(exact_pass);
      if (exact_pass) { b.val = -INFINITY; b.idx = 0x7fffffff; }
    }
    if (exact_pass)
      for (int v = v0 + threadIdx.x; v < v1; v += kSampleThreads) take(v, *reinterpret_cast<const uint4*>(row + v * 8));
    if (part == parts - 1)
      for (int c = nvec * 8 + threadIdx.x; c < p.vocab; c += kSampleThreads) consider(c, row[c]);
  } else {
    const int c0 = static_cast<int>(static_cast<int64_t>(p.vocab) * part / parts);
    const int c1 = static_cast<int>(static_cast<int64_t>(p.vocab) * (part + 1) / parts);
    for (int c = c0 + threadIdx.x; c < c1; c += kSampleThreads) consider(c, row[c]);
  }
  b = block_argmax(b);
  if (parts > 1) {
    if (threadIdx.x == 0) slice_best = b;
    cluster.sync();
    if (part == 0 && threadIdx.x < 32) {
      Best o{-INFINITY, 0x7fffffff};
      if (threadIdx.x < parts) o = *cluster.map_shared_rank(&slice_best, threadIdx.x);
#pragma unroll
      for (int s = 4; s > 0; s >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, o.val, s);
        const int oi = __shfl_xor_sync(0xffffffffu, o.idx, s);
        if (better(ov, oi, o.val, o.idx)) { o.val = ov; o.idx = oi; }
      }
      b = o;
    }
    cluster.sync();                                          // the slices' shared memory stays alive until it was read
    if (part != 0) return;
  }
  if (threadIdx.x == 0) {
    if (b.idx == 0x7fffffff) b.idx = 0;                       // a row of -inf only: nothing ever exceeded the start value
    p.out[r] = b.idx;
    if (p.scatter_table != nullptr) p.scatter_table[p.scatter_index[r]] = b.idx;
  }
}

constexpr int kKeptCap = 4096;       // kept (top-k) entries that the random path holds in shared memory
constexpr int kRankCap = 1024;       // lists up to this length are ranked by pairwise comparison

__global__ void __launch_bounds__(kSampleThreads, 2) sample_topk_gumbel_kernel(const SampleParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int parts = static_cast<int>(cluster.num_blocks()), part = static_cast<int>(cluster.block_rank());
  constexpr int NW = kSampleThreads / 32;
  __shared__ uint32_t hist_w[NW][256];                       // one histogram per warp: no contention between warps
  __shared__ uint32_t hist[256];
  __shared__ float mass[256];
  __shared__ uint32_t sel_s[2];                              // selected bin, entries needed inside it
  __shared__ float self_s[2];                                // nucleus: mass still needed, total mass
  __shared__ int32_t kept_col[kKeptCap];
  __shared__ uint16_t kept_bits[kKeptCap];
  __shared__ uint32_t n_kept_s;
  __shared__ float kept_w[kRankCap];                         // softmax weights of a short list
  __shared__ uint32_t cut_s;                                 // this slice's cut (read by the cluster)
  const int r = blockIdx.x / parts;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint16_t* row = p.logits + r * p.row_stride;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  const float temp = p.temperatures != nullptr ? p.temperatures[r] : 1.f;
  const bool scaled = p.temperatures != nullptr;
  const int k = p.top_k != nullptr ? p.top_k[r] : 0;
  const float top_p = p.top_p != nullptr ? p.top_p[r] : 1.f;
  const uint32_t k0 = static_cast<uint32_t>(p.seed), k1 = static_cast<uint32_t>(p.seed >> 32);
  const uint32_t o0 = static_cast<uint32_t>(p.offset), o1 = static_cast<uint32_t>(p.offset >> 32);
  auto emit = [&](int token) {                               // thread 0
    p.out[r] = token;
    if (p.scatter_table != nullptr) p.scatter_table[p.scatter_index[r]] = token;
  };
  auto gumbel_score = [&](int c, uint16_t bits) -> float {
    uint32_t rnd[4];
    philox4x32_10(static_cast<uint32_t>(c >> 2), static_cast<uint32_t>(r), o0, o1, k0, k1, rnd);
    const float u = __fmul_rn(__fadd_rn(static_cast<float>(rnd[c & 3] >> 9), 0.5f), 1.0f / 8388608.0f);
    float x = bits_to_float(bits);
    if (scaled) x = __fdiv_rn(x, temp);
    return __fsub_rn(x, logf(-logf(u)));
  };

  // ---- the usual case: a short list that is sure to hold the row's top k ---------------------------------------
  // (the whole cluster sees the same k, so either every CTA takes this branch or only the first one goes on)
  const bool windowed = k > 0 && k < p.vocab;
  if (!windowed && part != 0) return;
  bool have_list = false;                                    // the first CTA's list holds at least k entries, among them the top k
  if (windowed) {
    if (threadIdx.x == 0) n_kept_s = 0;                        // (visible to the cluster before anybody adds to it: sync below)
    // 1. per thread the maxima of the even and of the odd columns it reads (packed bf16 compares, 1-2
    //    instructions per two logits)
    __nv_bfloat162 m2 = __floats2bfloat162_rn(-INFINITY, -INFINITY);
    for_each_word_slice(row, p.vocab, vec_ok, part, parts,
                        [&](int, uint32_t w) { m2 = __hmax2_nan(m2, *reinterpret_cast<const __nv_bfloat162*>(&w)); });
    // 2. the k-th largest of the CTA's 2 * kSampleThreads sub-maxima, by two radix passes over their 16-bit keys.
    //    A NaN (its key lies above +inf's) or a k beyond the number of sub-maxima sends the row the general way.
    const uint32_t key_lo = sort_key(__bfloat16_as_ushort(__low2bfloat16(m2)));
    const uint32_t key_hi = sort_key(__bfloat16_as_ushort(__high2bfloat16(m2)));
    const bool odd = (key_lo > 0xff80u) || (key_hi > 0xff80u) || k > 2 * kSampleThreads;
    // the bin (counted from the top) in which the running count reaches `need`, and what is still needed inside it
    auto pick_bin = [&](uint32_t need) {                       // warp 0; result in sel_s
      uint32_t c[8], mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * lane - j]; mine += c[j]; }
      uint32_t incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const uint32_t first = __ffs(__ballot_sync(0xffffffffu, incl >= need)) - 1;   // need <= total: some lane qualifies
      if (lane == static_cast<int>(first)) {
        uint32_t left = need - (incl - mine);
        int j = 0;
        while (j < 7 && c[j] < left) { left -= c[j]; ++j; }
        sel_s[0] = 255 - 8 * lane - j; sel_s[1] = left;
      }
    };
    for (int i = threadIdx.x; i < 256; i += kSampleThreads) hist[i] = 0;
    const bool any_odd = __syncthreads_or(odd);
    uint32_t cut = 0;                                          // entries with key >= cut go on the list
    if (!any_odd) {
      atomicAdd(&hist[key_lo >> 8], 1u);
      atomicAdd(&hist[key_hi >> 8], 1u);
      __syncthreads();
      if (warp == 0) pick_bin(static_cast<uint32_t>(k));
      __syncthreads();
      const uint32_t hi_bin = sel_s[0], need_hi = sel_s[1];
      for (int i = threadIdx.x; i < 256; i += kSampleThreads) hist[i] = 0;
      __syncthreads();
      if ((key_lo >> 8) == hi_bin) atomicAdd(&hist[key_lo & 0xffu], 1u);
      if ((key_hi >> 8) == hi_bin) atomicAdd(&hist[key_hi & 0xffu], 1u);
      __syncthreads();
      if (warp == 0) pick_bin(need_hi);
      __syncthreads();
      cut = (hi_bin << 8) | sel_s[0];
      __syncthreads();                                         // sel_s is free again
    }
    // The row has at least k entries that reach ANY slice's cut, so the largest of the cuts serves every slice
    // and the lists of all slices together hold about k entries instead of k per slice.
    if (parts > 1) {
      if (threadIdx.x == 0) cut_s = any_odd ? 0xffffffffu : cut;
      cluster.sync();
      if (threadIdx.x < 32) {
        uint32_t c = 0;
        if (threadIdx.x < parts) c = *cluster.map_shared_rank(&cut_s, threadIdx.x);
        c = __reduce_max_sync(0xffffffffu, c);
        if (threadIdx.x == 0) sel_s[0] = c;
      }
      __syncthreads();
      cut = sel_s[0];
      __syncthreads();
    }
    const bool give_up = parts > 1 ? cut == 0xffffffffu : any_odd;   // some slice could not make a cut: the general way
    if (!give_up) {
      // 3. the entries that reach the cut go into this CTA's list ...
      const __nv_bfloat16 t1 = __ushort_as_bfloat16(key_to_bits(cut));
      const __nv_bfloat162 t2 = __halves2bfloat162(t1, t1);
      auto push = [&](int c, uint16_t bits) {
        if (c >= p.vocab) return;                             // the pad of an odd last column
        const uint32_t slot = atomicAdd(&n_kept_s, 1u);
        if (slot < kKeptCap) { kept_col[slot] = c; kept_bits[slot] = bits; }
      };
      // Only a thread whose own sub-maxima reach the cut has such entries among its words: about k of the
      // 2 * kSampleThreads sub-maxima do.  Those threads put their index on a list and the whole CTA then reads
      // the listed threads' words again (from L2), a handful of loads per thread in one round trip, instead of
      // every thread walking its own forty words four at a time.
      auto scan = [&](int c, uint32_t w) {
        const uint32_t ge = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w), t2);
        if (ge == 0u) return;
        if (ge & 0xffffu) push(c, static_cast<uint16_t>(w & 0xffffu));
        if (ge >> 16) push(c + 1, static_cast<uint16_t>(w >> 16));
      };
      const bool mine = __hge2_mask(m2, t2) != 0u;
      if (vec_ok) {
        uint16_t* qlist = reinterpret_cast<uint16_t*>(hist_w);  // (the per-warp histograms are not in use here)
        if (threadIdx.x == 0) sel_s[1] = 0u;
        __syncthreads();
        if (mine) qlist[atomicAdd(&sel_s[1], 1u)] = static_cast<uint16_t>(threadIdx.x);
        __syncthreads();
        const int n_q = static_cast<int>(sel_s[1]);
        const int nvec = p.vocab / 8;
        const int v0 = static_cast<int>(static_cast<int64_t>(nvec) * part / parts);
        const int v1 = static_cast<int>(static_cast<int64_t>(nvec) * (part + 1) / parts);
        const int per = (v1 - v0 + kSampleThreads - 1) / kSampleThreads;      // words of one thread
        const int items = n_q * per;
        for (int it = threadIdx.x; it < items; it += 4 * kSampleThreads) {
          uint4 w[4];
          int v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int item = it + u * kSampleThreads;
            v[u] = v1;
            if (item < items) {
              const int qi = item / per, i = item - qi * per;
              v[u] = v0 + static_cast<int>(qlist[qi]) + i * kSampleThreads;
            }
            if (v[u] < v1) w[u] = *reinterpret_cast<const uint4*>(row + v[u] * 8);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v[u] < v1) { scan(v[u] * 8, w[u].x); scan(v[u] * 8 + 2, w[u].y); scan(v[u] * 8 + 4, w[u].z); scan(v[u] * 8 + 6, w[u].w); }
        }
        if (mine && part == parts - 1) {                       // the columns past the last whole 16-byte word
          for (int c = nvec * 8 + 2 * threadIdx.x; c < p.vocab; c += 2 * kSampleThreads) {
            const uint32_t lo = row[c], hi = c + 1 < p.vocab ? row[c + 1] : 0xff80u;
            scan(c, lo | (hi << 16));
          }
        }
      } else if (mine) {
        for_each_word_slice(row, p.vocab, vec_ok, part, parts, scan);
      }
    }
    __syncthreads();
    // 4. ... and from there into the first CTA's list, one reservation per CTA
    if (parts > 1) {
      if (part != 0 && !give_up) {
        const uint32_t n_local = n_kept_s;
        uint32_t* n_remote = cluster.map_shared_rank(&n_kept_s, 0);
        int32_t* col_remote = cluster.map_shared_rank(kept_col, 0);
        uint16_t* bits_remote = cluster.map_shared_rank(kept_bits, 0);
        if (threadIdx.x == 0) sel_s[1] = atomicAdd(n_remote, n_local);
        __syncthreads();
        const uint32_t base = sel_s[1];
        for (uint32_t i = threadIdx.x; i < n_local && i < kKeptCap; i += kSampleThreads) {
          const uint32_t slot = base + i;
          if (slot < kKeptCap) { col_remote[slot] = kept_col[i]; bits_remote[slot] = kept_bits[i]; }
        }
      }
      cluster.sync();                                        // the first CTA's list is complete; the others are done
      if (part != 0) return;
    }
    const uint32_t n = n_kept_s;
    have_list = !give_up && n >= static_cast<uint32_t>(k) && n <= kKeptCap;
    if (have_list && n <= kRankCap) {
      // 5. ranks and masses by pairwise comparison.  Keys replace the raw bits (-0 becomes +0: same value).
      uint32_t km = 0;
      for (uint32_t i = threadIdx.x; i < n; i += kSampleThreads) {
        const uint32_t key = sort_key(kept_bits[i]);
        kept_bits[i] = static_cast<uint16_t>(key);
        km = key > km ? key : km;
      }
      km = __reduce_max_sync(0xffffffffu, km);
      if (lane == 0) hist[warp] = km;
      __syncthreads();
      if (threadIdx.x < 32) {
        const uint32_t m = __reduce_max_sync(0xffffffffu, threadIdx.x < NW ? hist[threadIdx.x] : 0u);
        if (threadIdx.x == 0) sel_s[0] = m;
      }
      __syncthreads();
      float xmax = bits_to_float(key_to_bits(sel_s[0]));
      if (scaled) xmax = __fdiv_rn(xmax, temp);
      for (uint32_t i = threadIdx.x; i < n; i += kSampleThreads) {
        float x = bits_to_float(key_to_bits(kept_bits[i]));
        if (scaled) x = __fdiv_rn(x, temp);
        kept_w[i] = expf(x - xmax);
      }
      __syncthreads();
      // entry i stays in the top k iff fewer than k entries are larger; it stays in the nucleus iff the mass of
      // the larger entries is below top_p of the kept mass (entries equal to the last one admitted stay too)
      constexpr int PER = (kRankCap + kSampleThreads - 1) / kSampleThreads;
      uint32_t cnt[PER];
      float above[PER], kept_mass = 0.f;
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const uint32_t i = threadIdx.x + u * kSampleThreads;
        cnt[u] = 0; above[u] = 0.f;
        if (i < n) {
          const uint32_t key = kept_bits[i];
          for (uint32_t j = 0; j < n; ++j) {
            const bool larger = kept_bits[j] > key;
            cnt[u] += larger ? 1u : 0u;
            above[u] += larger ? kept_w[j] : 0.f;
          }
          if (cnt[u] < static_cast<uint32_t>(k)) kept_mass += kept_w[i];
        }
      }
      float need = INFINITY;
      if (top_p < 1.f) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) kept_mass += __shfl_xor_sync(0xffffffffu, kept_mass, o);
        if (lane == 0) mass[warp] = kept_mass;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) total += mass[w];
        need = top_p * total;
      }
      Best b{-INFINITY, 0x7fffffff};
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const uint32_t i = threadIdx.x + u * kSampleThreads;
        if (i < n && cnt[u] < static_cast<uint32_t>(k) && (above[u] < need || cnt[u] == 0u)) {
          const int c = kept_col[i];
          const float score = gumbel_score(c, key_to_bits(kept_bits[i]));
          if (better(score, c, b.val, b.idx)) { b.val = score; b.idx = c; }
        }
      }
      b = block_argmax(b);
      if (threadIdx.x == 0) emit(b.idx);
      return;
    }
    __syncthreads();
  }

  // ---- the general way: radix selection over the whole row (first CTA of the cluster only) -----------------
  // counts of one byte of the key (entries for which keep(key) holds), summed into hist; over the row or,
  // once the candidates sit in shared memory, over those
  auto count_pass = [&](bool from_kept, auto bin_of, auto keep) {
    for (int i = threadIdx.x; i < NW * 256; i += kSampleThreads) (&hist_w[0][0])[i] = 0;
    __syncthreads();
    auto add = [&](uint16_t bits) {
      const uint32_t key = sort_key(bits);
      if (keep(key)) atomicAdd(&hist_w[warp][bin_of(key)], 1u);
    };
    if (from_kept) {
      const int n = static_cast<int>(n_kept_s);
      for (int i = threadIdx.x; i < n; i += kSampleThreads) add(kept_bits[i]);
    } else {
      for_each_logit(row, p.vocab, vec_ok, [&](int, uint16_t bits) { add(bits); });
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kSampleThreads) {
      uint32_t n = 0;
#pragma unroll
      for (int w = 0; w < NW; ++w) n += hist_w[w][i];
      hist[i] = n;
    }
    __syncthreads();
  };
  // the key of the k-th largest entry by two radix passes (high byte, then low byte inside its bin)
  auto kth_key = [&](bool from_kept) -> uint32_t {
    count_pass(from_kept, [](uint32_t key) { return key >> 8; }, [](uint32_t) { return true; });
    if (threadIdx.x == 0) {
      uint32_t need = k, bin = 0;
      for (int i = 255; i >= 0; --i) {
        if (hist[i] >= need) { bin = i; break; }
        need -= hist[i];
      }
      sel_s[0] = bin; sel_s[1] = need;
    }
    __syncthreads();
    const uint32_t hi_bin = sel_s[0], need_hi = sel_s[1];
    __syncthreads();
    count_pass(from_kept, [](uint32_t key) { return key & 0xffu; }, [&](uint32_t key) { return (key >> 8) == hi_bin; });
    if (threadIdx.x == 0) {
      uint32_t need = need_hi, bin = 0;
      for (int i = 255; i >= 0; --i) {
        if (hist[i] >= need) { bin = i; break; }
        need -= hist[i];
      }
      sel_s[0] = bin;
    }
    __syncthreads();
    const uint32_t key = (hi_bin << 8) | sel_s[0];
    __syncthreads();
    return key;
  };
  // entries with key >= lo move into shared memory (all of them counted, the first kKeptCap stored)
  auto gather = [&](uint32_t lo) {
    if (threadIdx.x == 0) n_kept_s = 0;
    __syncthreads();
    for_each_logit(row, p.vocab, vec_ok, [&](int c, uint16_t bits) {
      if (sort_key(bits) < lo) return;
      const uint32_t slot = atomicAdd(&n_kept_s, 1u);
      if (slot < kKeptCap) { kept_col[slot] = c; kept_bits[slot] = bits; }
    });
    __syncthreads();
  };

  uint32_t thresh = 0;                                       // keep keys >= thresh
  bool compact = false;                                      // the candidates sit in shared memory
  if (windowed && have_list) {
    thresh = kth_key(true);                                  // (a list too long to rank pairwise)
    compact = true;
  } else if (windowed) {
    // the kept entries (k of them, plus ties at the threshold) into shared memory if they fit
    thresh = kth_key(false);
    gather(thresh);
    compact = n_kept_s <= kKeptCap;
  }
  const int n_kept = compact ? static_cast<int>(n_kept_s) : 0;
  // f(column, bits) for every entry with key >= thresh
  auto for_each_kept = [&](auto f) {
    if (compact) {
      for (int i = threadIdx.x; i < n_kept; i += kSampleThreads)
        if (sort_key(kept_bits[i]) >= thresh) f(kept_col[i], kept_bits[i]);
    } else {
      for_each_logit(row, p.vocab, vec_ok, [&](int c, uint16_t bits) {
        if (sort_key(bits) >= thresh) f(c, bits);
      });
    }
  };

  if (top_p < 1.f) {
    // nucleus: the smallest set of the most likely kept tokens whose probability mass reaches top_p,
    // found like the top-k threshold but with histograms of exp(x - max) instead of counts
    Best mx{-INFINITY, 0x7fffffff};
    for_each_kept([&](int c, uint16_t bits) {
      float x = bits_to_float(bits);
      if (scaled) x = __fdiv_rn(x, temp);
      if (better(x, c, mx.val, mx.idx)) { mx.val = x; mx.idx = c; }
    });
    mx = block_argmax(mx);
    if (threadIdx.x == 0) self_s[1] = mx.val;
    for (int i = threadIdx.x; i < 256; i += kSampleThreads) mass[i] = 0.f;
    __syncthreads();
    const float xmax = self_s[1];
    __syncthreads();
    auto weight = [&](uint16_t bits) {
      float x = bits_to_float(bits);
      if (scaled) x = __fdiv_rn(x, temp);
      return expf(x - xmax);
    };
    for_each_kept([&](int, uint16_t bits) { atomicAdd(&mass[sort_key(bits) >> 8], weight(bits)); });
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int i = 0; i < 256; ++i) total += mass[i];
      float need = top_p * total;
      uint32_t bin = thresh >> 8;
      for (int i = 255; i >= static_cast<int>(thresh >> 8); --i) {
        if (mass[i] >= need) { bin = i; break; }
        need -= mass[i];
      }
      sel_s[0] = bin; self_s[0] = need;
    }
    __syncthreads();
    const uint32_t hi_bin = sel_s[0];
    const float need_hi = self_s[0];
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kSampleThreads) mass[i] = 0.f;
    __syncthreads();
    for_each_kept([&](int, uint16_t bits) {
      const uint32_t key = sort_key(bits);
      if ((key >> 8) == hi_bin) atomicAdd(&mass[key & 0xffu], weight(bits));
    });
    __syncthreads();
    if (threadIdx.x == 0) {
      float need = need_hi;
      uint32_t bin = 0;
      for (int i = 255; i >= 0; --i) {
        if (mass[i] >= need && mass[i] > 0.f) { bin = i; break; }
        need -= mass[i];
      }
      sel_s[0] = bin;
    }
    __syncthreads();
    const uint32_t nucleus = (hi_bin << 8) | sel_s[0];
    thresh = nucleus > thresh ? nucleus : thresh;
    __syncthreads();
  }

  Best b{-INFINITY, 0x7fffffff};
  // (the compacted list was made with the top-k threshold; the nucleus may have raised it since)
  uint32_t rnd[4];
  int rnd_group = -1;                                        // a whole-row pass meets the 4 columns of a Philox block in turn
  for_each_kept([&](int c, uint16_t bits) {
    if (sort_key(bits) < thresh) return;
    if ((c >> 2) != rnd_group) {
      rnd_group = c >> 2;
      philox4x32_10(static_cast<uint32_t>(rnd_group), static_cast<uint32_t>(r), o0, o1, k0, k1, rnd);
    }
    const float u = __fmul_rn(__fadd_rn(static_cast<float>(rnd[c & 3] >> 9), 0.5f), 1.0f / 8388608.0f);
    float x = bits_to_float(bits);
    if (scaled) x = __fdiv_rn(x, temp);
    const float score = __fsub_rn(x, logf(-logf(u)));
    if (better(score, c, b.val, b.idx)) { b.val = score; b.idx = c; }
  });
  b = block_argmax(b);
  if (threadIdx.x == 0) emit(b.idx);
}

}  // namespace mvb

extern "C" int mvb_sample(const void* logits, int64_t row_stride, int num_rows, int vocab,
                          const float* temperatures, const int32_t* top_k, const float* top_p, uint64_t seed,
                          uint64_t offset, int64_t* out, int64_t* scatter_table, const int32_t* scatter_index, int32_t* dev_status,
                          void* stream) {
  using namespace mvb;
  (void)dev_status;
  if (!logits || !out || num_rows < 0 || vocab <= 0 || row_stride < vocab) return kInvalidArgument;
  if ((scatter_table == nullptr) != (scatter_index == nullptr)) return kInvalidArgument;
  if (num_rows == 0) return kOk;
  SampleParams p{static_cast<const uint16_t*>(logits), row_stride, vocab, temperatures, top_k, top_p, seed, offset,
                 out, scatter_table, scatter_index};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // A cluster of up to 8 CTAs per row when the batch is small.  Greedy rows are one streaming pass: enough CTAs
  // for two per SM.  The random path pays for every extra slice with a longer candidate list and two cluster
  // barriers, so it stops splitting once half the SMs have a CTA.
  const bool greedy = top_k == nullptr && top_p == nullptr;
  const int64_t enough = greedy ? 2 * sm_count() : (sm_count() + 1) / 2;
  int parts = 1;
  while (parts < 8 && static_cast<int64_t>(num_rows) * parts < enough) parts *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(num_rows) * parts);
  cfg.blockDim = dim3(kSampleThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = parts; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = greedy ? cudaLaunchKernelEx(&cfg, sample_greedy_kernel, p)
                                 : cudaLaunchKernelEx(&cfg, sample_topk_gumbel_kernel, p);
  return err == cudaSuccess ? kOk : kLaunchFailed;
}
