// Device-side batch packing: per-sequence facts -> per-token tensors of the Context contract.
//
// The host uploads O(num_seqs + num_blocks + new tokens) int32 values in one buffer; these
// kernels expand them into cu_seqlens / positions / slot_mapping / input_ids / block table
// with a block-wide prefix sum and a per-token binary search (integer work, HBM/latency bound;
// outputs are bit-exact restatements of the host loops they replace).
#include "common.cuh"
#include "scan.cuh"
#include "mini_vllm_b200.h"

namespace mvb {

constexpr int kPackThreads = 256;

struct PackPrefillParams {
  const int32_t *seq_len, *cached_len, *blk_off, *blocks_flat, *new_tokens;
  int num_seqs, num_tokens, table_width, block_size;
  int64_t *input_ids, *positions;
  int32_t *slot_mapping, *cu_q, *cu_k, *block_table;
  int* dev_status;
};

__global__ void __launch_bounds__(kPackThreads) pack_prefill_kernel(const PackPrefillParams p) {
  extern __shared__ int32_t cu_q_s[];                       // [num_seqs + 1]
  block_exclusive_scan<kPackThreads>([&](int i) { return p.seq_len[i] - p.cached_len[i]; }, p.num_seqs, cu_q_s);
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i <= p.num_seqs; i += kPackThreads) p.cu_q[i] = cu_q_s[i];
    block_exclusive_scan<kPackThreads>([&](int i) { return p.seq_len[i]; }, p.num_seqs, p.cu_k);
    if (threadIdx.x == 0 && cu_q_s[p.num_seqs] != p.num_tokens) report(p.dev_status, kDevBadLength, cu_q_s[p.num_seqs]);
  }
  const int stride = gridDim.x * kPackThreads;
  for (int t = blockIdx.x * kPackThreads + threadIdx.x; t < p.num_tokens; t += stride) {
    // last s with cu_q[s] <= t (skips sequences that contribute no query token)
    int lo = 0, hi = p.num_seqs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cu_q_s[mid] <= t) lo = mid; else hi = mid;
    }
    const int s = lo;
    const int pos = p.cached_len[s] + (t - cu_q_s[s]);
    p.input_ids[t] = p.new_tokens[t];
    p.positions[t] = pos;
    const int b0 = p.blk_off[s], nb = p.blk_off[s + 1] - b0;
    const int bi = pos / p.block_size;
    int32_t slot = -1;
    if (bi < nb) slot = p.blocks_flat[b0 + bi] * p.block_size + (pos - bi * p.block_size);
    p.slot_mapping[t] = slot;
  }
  if (p.block_table != nullptr) {
    const int total = p.num_seqs * p.table_width;
    for (int e = blockIdx.x * kPackThreads + threadIdx.x; e < total; e += stride) {
      const int s = e / p.table_width, c = e - s * p.table_width;
      const int b0 = p.blk_off[s], nb = p.blk_off[s + 1] - b0;
      p.block_table[e] = c < nb ? p.blocks_flat[b0 + c] : -1;
    }
  }
}

struct PackDecodeParams {
  const int32_t *seq_len, *blk_off, *blocks_flat, *host_tokens;
  const int64_t* prev_sampled;
  const int32_t* src_index;
  int num_seqs, padded_seqs, table_width, block_size;
  int64_t table_stride;
  int64_t *input_ids, *positions;
  int32_t *slot_mapping, *cache_seqlens, *block_table;
  int* dev_status;
};

__global__ void __launch_bounds__(kPackThreads) pack_decode_kernel(const PackDecodeParams p) {
  const int stride = gridDim.x * kPackThreads;
  const int gid = blockIdx.x * kPackThreads + threadIdx.x;
  for (int b = gid; b < p.padded_seqs; b += stride) {
    if (b >= p.num_seqs) {                                   // graph padding row
      p.input_ids[b] = 0; p.positions[b] = 0; p.slot_mapping[b] = -1; p.cache_seqlens[b] = 0;
      continue;
    }
    const int n = p.seq_len[b];
    const int b0 = p.blk_off[b], nb = p.blk_off[b + 1] - b0;
    int64_t tok;
    if (p.prev_sampled != nullptr && p.src_index != nullptr && p.src_index[b] >= 0) tok = p.prev_sampled[p.src_index[b]];
    else tok = p.host_tokens[b];
    p.input_ids[b] = tok;
    p.positions[b] = n - 1;
    p.cache_seqlens[b] = n;
    int32_t slot = -1;
    if (nb > 0 && n > (nb - 1) * p.block_size && n <= nb * p.block_size) {
      slot = p.blocks_flat[b0 + nb - 1] * p.block_size + (n - (nb - 1) * p.block_size) - 1;
    } else {
      report(p.dev_status, kDevBadLength, b);
    }
    p.slot_mapping[b] = slot;
  }
  const int total = p.padded_seqs * p.table_width;
  for (int e = gid; e < total; e += stride) {
    const int s = e / p.table_width, c = e - s * p.table_width;
    int32_t val = -1;
    if (s < p.num_seqs) {
      const int b0 = p.blk_off[s], nb = p.blk_off[s + 1] - b0;
      if (c < nb) val = p.blocks_flat[b0 + c];
    }
    p.block_table[s * p.table_stride + c] = val;
  }
}

}  // namespace mvb

extern "C" int mvb_pack_prefill(const int32_t* seq_len, const int32_t* cached_len, const int32_t* blk_off,
                                const int32_t* blocks_flat, const int32_t* new_tokens, int num_seqs,
                                int num_tokens, int table_width, int block_size, int64_t* input_ids,
                                int64_t* positions, int32_t* slot_mapping, int32_t* cu_seqlens_q,
                                int32_t* cu_seqlens_k, int32_t* block_table, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (num_seqs <= 0 || num_tokens < 0 || block_size <= 0 || table_width < 0) return kInvalidArgument;
  if (!seq_len || !cached_len || !blk_off || !cu_seqlens_q || !cu_seqlens_k) return kInvalidArgument;
  if (num_tokens > 0 && (!new_tokens || !input_ids || !positions || !slot_mapping)) return kInvalidArgument;
  if (block_table != nullptr && table_width == 0) return kInvalidArgument;
  const size_t smem = static_cast<size_t>(num_seqs + 1) * sizeof(int32_t);
  if (smem > 200 * 1024) return kUnsupportedShape;
  PackPrefillParams p{seq_len, cached_len, blk_off, blocks_flat, new_tokens, num_seqs, num_tokens, table_width,
                      block_size, input_ids, positions, slot_mapping, cu_seqlens_q, cu_seqlens_k, block_table,
                      dev_status};
  int64_t work = num_tokens;
  if (block_table != nullptr && static_cast<int64_t>(num_seqs) * table_width > work)
    work = static_cast<int64_t>(num_seqs) * table_width;
  int blocks = static_cast<int>((work + kPackThreads - 1) / kPackThreads);
  blocks = blocks < 1 ? 1 : (blocks > 148 * 4 ? 148 * 4 : blocks);
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(pack_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return kLaunchFailed;
  }
  pack_prefill_kernel<<<blocks, kPackThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

extern "C" int mvb_pack_decode(const int32_t* seq_len, const int32_t* blk_off, const int32_t* blocks_flat,
                               const int32_t* host_tokens, const int64_t* prev_sampled, const int32_t* src_index,
                               int num_seqs, int padded_seqs, int table_width, int64_t table_stride,
                               int block_size, int64_t* input_ids, int64_t* positions, int32_t* slot_mapping,
                               int32_t* cache_seqlens, int32_t* block_table, int32_t* dev_status, void* stream) {
  using namespace mvb;
  if (num_seqs <= 0 || padded_seqs < num_seqs || block_size <= 0 || table_width <= 0 || table_stride < table_width)
    return kInvalidArgument;
  if (!seq_len || !blk_off || !blocks_flat || !input_ids || !positions || !slot_mapping || !cache_seqlens ||
      !block_table)
    return kInvalidArgument;
  if (!host_tokens && !(prev_sampled && src_index)) return kInvalidArgument;
  PackDecodeParams p{seq_len, blk_off, blocks_flat, host_tokens, prev_sampled, src_index, num_seqs, padded_seqs,
                     table_width, block_size, table_stride, input_ids, positions, slot_mapping, cache_seqlens,
                     block_table, dev_status};
  const int64_t work = static_cast<int64_t>(padded_seqs) * table_width;
  int blocks = static_cast<int>((work + kPackThreads - 1) / kPackThreads);
  blocks = blocks < 1 ? 1 : (blocks > 148 * 4 ? 148 * 4 : blocks);
  pack_decode_kernel<<<blocks, kPackThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}
