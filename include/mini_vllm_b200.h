/*
 * C ABI of libmini_vllm_b200.so: the B200 (sm_100a) kernels for mini-vllm's ragged
 * continuous-batching attention path.
 *
 * Conventions for every entry point
 *   - All data pointers are DEVICE pointers owned by the caller (typically PyTorch tensors
 *     kept alive until the stream reaches the launch).  Nothing here allocates, frees,
 *     synchronises or throws; work is enqueued on `stream` (a cudaStream_t passed as void*).
 *   - Return value: 0 on success, a negative mvb_status for an argument error found on the
 *     host (nothing is launched in that case).
 *   - `dev_status` (optional, may be NULL) is a device int32[4] the caller zeroes; a kernel
 *     that meets an out-of-range slot / block id / position, or whose bounded wait runs out,
 *     records {code, detail, block, thread} there, skips the access and carries on.
 *   - bf16 tensors are passed as void*; the last dimension (head_dim) is contiguous and
 *     heads are contiguous (stride head_dim); only the token (row) stride is free.
 *   - KV pool layout per layer: [num_blocks, block_size, num_kv_heads, head_dim] bf16,
 *     contiguous, the layout the reference allocates in
 *     minivllm/executor/executor.py:51-60.  A slot is block_id * block_size + offset.
 *
 * Reference citations are paths inside w4096/mini-vllm.
 */
#ifndef MINI_VLLM_B200_H_
#define MINI_VLLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum mvb_status {
  MVB_OK = 0,
  MVB_INVALID_ARGUMENT = -1,
  MVB_UNSUPPORTED_SHAPE = -2,
  MVB_LAUNCH_FAILED = -3,
  MVB_TENSOR_MAP_FAILED = -4,
  MVB_MISALIGNED = -5,
  MVB_NO_DRIVER_ENTRY = -6,
  MVB_SCRATCH_TOO_SMALL = -7
};

/* Library ABI version (bumped when a signature changes). */
int mvb_abi_version(void);
/* Human-readable name of a status code. */
const char* mvb_status_string(int status);

/*
 * Self-test of the kernels' bounded waits.  (No counterpart in the reference.)
 * Every wait inside the attention kernels is an mbarrier wait with an iteration limit; when it runs out
 * the kernel records {4 = wait timeout, detail, block, thread} in dev_status and returns instead of
 * hanging.  This entry runs that same wait, with `limit` polls (1..65536), on a barrier nothing arrives
 * at, so the status path can be exercised without disturbing a real kernel: after the stream has drained
 * dev_status[0] == 4 and dev_status[1] == limit.
 */
int mvb_selftest_wait_timeout(int32_t* dev_status, int limit, void* stream);

/*
 * Prefill batch packing on the device.
 * Replaces Executor._build_prefill_input (minivllm/executor/executor.py:81-127) and
 * Executor._build_block_table (:156-163): from per-sequence facts it expands
 *   input_ids[t], positions[t] = cached + i, slot_mapping[t] = blocks[pos/bs]*bs + pos%bs,
 *   cu_seqlens_q / cu_seqlens_k (exclusive prefix sums, int32 [num_seqs+1]) and, when
 *   block_table != NULL, the [num_seqs, table_width] table right-padded with -1.
 * Inputs (device int32): seq_len[num_seqs] (full length n), cached_len[num_seqs],
 *   blk_off[num_seqs+1] (exclusive prefix sum of per-sequence block counts),
 *   blocks_flat[blk_off[num_seqs]], new_tokens[num_tokens] (the uncached suffixes, concatenated).
 * A token whose block index is beyond its sequence's block list (warm-up requests own no
 * blocks, executor.py:62-78) gets slot -1.
 */
int mvb_pack_prefill(const int32_t* seq_len, const int32_t* cached_len, const int32_t* blk_off,
                     const int32_t* blocks_flat, const int32_t* new_tokens, int num_seqs, int num_tokens,
                     int table_width, int block_size, int64_t* input_ids, int64_t* positions,
                     int32_t* slot_mapping, int32_t* cu_seqlens_q, int32_t* cu_seqlens_k, int32_t* block_table,
                     int32_t* dev_status, void* stream);

/*
 * Decode batch packing on the device, written straight into (slices of) the CUDA-graph
 * runner's static buffers.
 * Replaces Executor._build_decode_input (minivllm/executor/executor.py:130-153) and the staging
 * copies of CudaGraphRunner.replay (minivllm/executor/graph.py:64-70).
 * For row b < num_seqs: input_ids = token, positions = n-1, cache_seqlens = n,
 *   slot = last_block*bs + (n - (nblk-1)*bs) - 1, block_table[b, :table_width] = blocks, pad -1.
 * Rows num_seqs..padded_seqs-1 are padding: input_ids 0, positions 0, slot -1, cache_seqlens 0,
 *   block table row -1.
 * The token of row b is prev_sampled[src_index[b]] when prev_sampled != NULL and
 * src_index[b] >= 0 (the previous step's sampler output, still on the device), else
 * host_tokens[b].
 * block_table has row stride table_stride (>= table_width) elements.
 */
int mvb_pack_decode(const int32_t* seq_len, const int32_t* blk_off, const int32_t* blocks_flat,
                    const int32_t* host_tokens, const int64_t* prev_sampled, const int32_t* src_index,
                    int num_seqs, int padded_seqs, int table_width, int64_t table_stride, int block_size,
                    int64_t* input_ids, int64_t* positions, int32_t* slot_mapping, int32_t* cache_seqlens,
                    int32_t* block_table, int32_t* dev_status, void* stream);

/*
 * Fused rotary embedding + paged KV-cache write.
 * Replaces RotaryEmbedding.forward (minivllm/models/layers/rotary.py:49-71) followed by
 * store_kvcache (minivllm/models/layers/attention.py:13-43).
 *   q [num_tokens, num_q_heads, head_dim] bf16, row stride q_row_stride elements: rotated in place.
 *   k [num_tokens, num_kv_heads, head_dim]: rotated; written to k_cache at slot_mapping[t]
 *     (skipped when the slot is -1 or slot_mapping == NULL) and, if k_in_place != 0, back into k.
 *   v: copied to v_cache at the same slot.
 *   cos_sin [max_pos, head_dim] fp32 = cat(cos, sin) as built by rotary.py:32-47; NULL disables
 *     the rotation (plain store_kvcache).  Arithmetic is fp32 with separately rounded products,
 *     one rounding to bf16, so results are bit-identical to the eager reference.
 * head_dim must be a multiple of 16; k_cache/v_cache may be NULL only with slot_mapping NULL.
 */
int mvb_rope_kv_write(void* q, int64_t q_row_stride, void* k, int64_t k_row_stride, const void* v,
                      int64_t v_row_stride, const int64_t* positions, const float* cos_sin, int64_t max_pos,
                      const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t num_slots,
                      int num_tokens, int num_q_heads, int num_kv_heads, int head_dim, int k_in_place,
                      int32_t* dev_status, void* stream);

/*
 * Per-head RMSNorm of q and k + rotary embedding + paged KV-cache write in one kernel.
 * Replaces the q_norm / k_norm / rotary_embedding / store_kvcache sequence of the model call-sites
 * (minivllm/models/models/qwen3.py:89-94, minivllm/models/models/gemma3.py:97-102).
 *   q, k, v are read where the projection left them (views of the packed qkv output are fine: only
 *   the row strides matter).  Each head row is normalised in fp32,
 *     y = x * rsqrt(mean(x^2) + eps) * w          (unit_offset == 0, nn.RMSNorm, qwen3.py:64-65)
 *     y = x * rsqrt(mean(x^2) + eps) * (1 + w)    (unit_offset != 0, gemma3.py:12-24)
 *   rounded to bf16 as the stand-alone norm would, rotated like mvb_rope_kv_write, and written: q in
 *   place, k to the cache slot (and in place if k_in_place), v to the cache slot.
 *   q_weight, k_weight: bf16 [head_dim].  head_dim / 16 must be a power of two (<= 32).
 * Results equal the unfused sequence up to the summation order of the squares (at most one bf16 ulp
 * on a few elements); use mvb_rope_kv_write where bit-exact KV contents are required.
 */
int mvb_qk_norm_rope_kv_write(void* q, int64_t q_row_stride, void* k, int64_t k_row_stride, const void* v,
                              int64_t v_row_stride, const void* q_weight, const void* k_weight, float eps,
                              int unit_offset, const int64_t* positions, const float* cos_sin, int64_t max_pos,
                              const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t num_slots,
                              int num_tokens, int num_q_heads, int num_kv_heads, int head_dim, int k_in_place,
                              int32_t* dev_status, void* stream);

/*
 * Paged decode attention (one query token per sequence), split along the context.
 * Replaces flash_attn_with_kvcache as called at minivllm/models/layers/attention.py:90-91.
 *
 * mvb_decode_workspace_bytes: size of the caller-supplied workspace for up to max_seqs rows.
 * mvb_decode_plan: one small launch per step (the plan depends only on cache_seqlens and the
 *   window, so every layer of a step shares it) that balances 16-token tiles over the
 *   persistent grid and records it in the workspace.
 * mvb_decode_attn: q [num_seqs, num_q_heads, head_dim] -> out (same shape, bf16).  Key j of
 *   sequence b is visible iff max(0, n-1-window_left) <= j < n with n = cache_seqlens[b]
 *   (window_left < 0: no window).  Rows with n == 0 (graph padding, graph.py:66-69) give zeros.
 *   Grid and pointers do not depend on data, so the launch sequence can be captured in a
 *   CUDA graph.  block_table is [num_seqs, table_width] with row stride table_stride.
 *   Supported: head_dim 128 or 256; num_q_heads/num_kv_heads <= 8; num_kv_heads in {1,2,4} or a
 *   multiple of 8 (head_dim 128) / 4 (head_dim 256); block_size a multiple of 16.
 *   The plan must have been made for the same cache_seqlens, window and head shape.
 */
size_t mvb_decode_workspace_bytes(int max_seqs, int num_q_heads, int head_dim);
int mvb_decode_plan(const int32_t* cache_seqlens, int num_seqs, int window_left, int num_q_heads,
                    int num_kv_heads, int head_dim, void* workspace, size_t workspace_bytes, void* stream);
/* Same plan, and the first block id of every CTA's range is looked up here once per step instead of by
 * every layer's attention kernel in front of its first TMA load (the table must be the one passed to
 * mvb_decode_attn). */
int mvb_decode_plan_with_table(const int32_t* cache_seqlens, const int32_t* block_table, int64_t table_stride,
                               int block_size, int num_seqs, int window_left, int num_q_heads, int num_kv_heads,
                               int head_dim, void* workspace, size_t workspace_bytes, void* stream);
int mvb_decode_attn(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                    int64_t num_blocks, int block_size, const int32_t* cache_seqlens,
                    const int32_t* block_table, int64_t table_stride, int table_width, int num_seqs,
                    int num_q_heads, int num_kv_heads, int head_dim, float scale, int window_left, void* out,
                    int64_t out_row_stride, void* workspace, size_t workspace_bytes, int32_t* dev_status,
                    void* stream);

/*
 * Decode attention for callers that cannot provide a workspace.  (No counterpart in the reference,
 * which lets PyTorch allocate whatever its attention library needs.)
 *
 * Meant for users who must not, or cannot, allocate device memory around this call: a process whose
 * GPU memory is fully parcelled out at start-up, a thin binding that can only pass on buffers it was
 * given, or a latency-critical loop that has to stay clear of cudaMalloc and its device-wide
 * synchronisation.  It computes exactly what mvb_decode_plan followed by mvb_decode_attn compute, but
 * keeps the plan, the partial results and the arrival counters in a MVB_STATIC_SCRATCH_BYTES array
 * that is part of the library image: each GPU that loads the library holds that memory until the
 * process ends.  Inputs and outputs are still the caller's.
 *
 *   - Limit: the scratch needed for (num_seqs, num_q_heads, head_dim) must fit the 8 MiB array.
 *     That covers 16 or 32 query heads of dimension 128 (or 4 to 16 of dimension 256) with
 *     thousands of sequences; 64 heads x 128 does not fit.  Larger requests return
 *     MVB_SCRATCH_TOO_SMALL and launch nothing.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside any stream capture.  No call allocates or frees memory.
 *   - All calls on a device share the one array.  Each call re-plans and clears what has to start
 *     at zero, so earlier contents do not matter, but two calls whose kernels overlap on the GPU
 *     (different streams) would race on it: keep them ordered.
 */
#define MVB_STATIC_SCRATCH_BYTES (8u << 20)
int mvb_decode_attn_static(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                           int64_t num_blocks, int block_size, const int32_t* cache_seqlens,
                           const int32_t* block_table, int64_t table_stride, int table_width, int num_seqs,
                           int num_q_heads, int num_kv_heads, int head_dim, float scale, int window_left,
                           void* out, int64_t out_row_stride, int32_t* dev_status, void* stream);

/*
 * Causal varlen prefill attention on the tcgen05 tensor cores.
 * Replaces flash_attn_varlen_func as called at minivllm/models/layers/attention.py:84-87.
 *   q [total_q, num_q_heads, head_dim]; sequence s owns rows cu_seqlens_q[s]..cu_seqlens_q[s+1].
 *   block_table == NULL: k, v are dense [total_k, num_kv_heads, head_dim] (row strides
 *     k_row_stride / v_row_stride; kv_rows = total_k) sliced by cu_seqlens_k.
 *   block_table != NULL: k, v are the paged pool (kv_rows = num_blocks*block_size slots,
 *     both row strides = num_kv_heads*head_dim) and keys 0..k_len-1 of sequence s are gathered
 *     through row s of the table (the prefix-cache case, attention.py:79-83).
 *   Query i of a sequence sits at position p = k_len - q_len + i and sees keys
 *   max(0, p - window_left) <= j <= p.
 * Supported: head_dim 128 or 256, any GQA ratio; with a block table, block_size a multiple of 128
 * (head_dim 128) or of 64 (head_dim 256), the kernel's KV tile, so that a tile never straddles blocks.
 */
int mvb_prefill_attn(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride, const void* v,
                     int64_t v_row_stride, int64_t kv_rows, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                     const int32_t* block_table, int64_t table_stride, int block_size, int num_seqs,
                     int total_q, int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                     float scale, int window_left, void* out, int64_t out_row_stride, int32_t* dev_status,
                     void* stream);

/*
 * The same launch with its work given as a list.  (No counterpart in the reference.)
 *   items: int32 [num_items, 2] on the device, one (sequence, query block) pair per work item; query block b of a
 *   sequence is its rows b*R .. b*R+R-1 with R = mvb_prefill_item_rows(...) (128 or 256, a property of the head
 *   layout).  The list must hold every query block of every sequence exactly once (rows of a block that is not
 *   listed are not written); its order is the order in which the GPU takes the work, so the caller lists the blocks
 *   with the most visible keys first.  Entries outside the batch are skipped.  num_items <= 65535.
 * Without the list mvb_prefill_attn launches a block index for every (sequence, block rank) up to the longest
 * sequence's block count; on a ragged batch most of those are empty and each costs a round trip to hand out
 * (config 3's prefill batch: 1920 indices for 872 items, 140 us; with the list, longest first: 112 us).
 * The host knows the lengths when it packs the step (Executor._build_prefill_input, executor.py:81-127), which is
 * where the list is built; results are bit-identical to mvb_prefill_attn.  A list that fills at least 85 % of
 * the grid (sequences of about one length) is not read: the grid form is run, which is then the faster one.
 */
int mvb_prefill_item_rows(int num_q_heads, int num_kv_heads, int head_dim);
int mvb_prefill_attn_items(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride, const void* v,
                           int64_t v_row_stride, int64_t kv_rows, const int32_t* cu_seqlens_q,
                           const int32_t* cu_seqlens_k, const int32_t* block_table, int64_t table_stride,
                           int block_size, int num_seqs, int total_q, int max_seqlen_q, int num_q_heads,
                           int num_kv_heads, int head_dim, float scale, int window_left, void* out,
                           int64_t out_row_stride, const int32_t* items, int num_items, int32_t* dev_status,
                           void* stream);

/*
 * Fused temperature / top-k / Gumbel-max sampler over the vocabulary.
 * Replaces Sampler.forward (minivllm/models/layers/sampler.py:9-31).
 *   logits [num_rows, vocab] bf16 (row stride in elements) -> out int64 [num_rows].
 *   top_k == NULL and top_p == NULL: greedy argmax of logits / temperature (lowest index wins ties), the
 *     reference's path when no top-k/top-p is requested (sampler.py:31).
 *   top_k != NULL or top_p != NULL: row r keeps every logit >= its top_k[r]-th largest
 *     (top_k[r] <= 0 keeps all), then, if top_p[r] < 1, the most likely of those until their
 *     softmax(logit / temperature) mass reaches top_p[r] (tokens tied with the last one are kept);
 *     it adds Gumbel noise from Philox4x32-10 keyed by (seed, offset, r, column) to
 *     logit / temperature and returns the argmax.  temperatures may be NULL (all 1).
 *   scatter_table/scatter_index (both or neither): the token of row r is also stored at
 *     scatter_table[scatter_index[r]], a per-request table the next decode packing reads its input
 *     tokens from (mvb_pack_decode's prev_sampled/src_index), so the sampled ids never have to visit
 *     the host between steps (the reference syncs on .tolist() every step, executor.py:193-195).
 */
int mvb_sample(const void* logits, int64_t row_stride, int num_rows, int vocab, const float* temperatures,
               const int32_t* top_k, const float* top_p, uint64_t seed, uint64_t offset, int64_t* out,
               int64_t* scatter_table, const int32_t* scatter_index, int32_t* dev_status, void* stream);

/*
 * lm_head and greedy sampling in one kernel: out[r] = argmax_n bf16(sum_k hidden_states[r, k] * weight[n, k]),
 * the lowest column winning ties.
 * Replaces, for requests without top-k / top-p (the reference's argmax path), logits = lm_head(hidden_states)
 * (minivllm/models/models/qwen3.py:215-219, gemma3.py:258-262) followed by Sampler.forward's
 * torch.argmax (minivllm/models/layers/sampler.py:31): a tcgen05 GEMM whose epilogue rounds each accumulator to
 * bf16 - the logit the unfused path would have stored - and keeps only the best (value, column) per row, so the
 * [num_rows, vocab] logits are never written or read back.  A positive temperature does not change an argmax
 * and is not needed here.
 *   hidden_states [num_rows, hidden] bf16 (row stride in elements), weight [vocab, hidden] bf16 (the lm_head /
 *   tied embedding matrix as stored); hidden a multiple of 64; rows 16-byte aligned.
 *   scratch: mvb_lm_head_argmax_scratch_bytes(max rows) bytes of device memory that the caller zeroes ONCE; every
 *   call leaves it zeroed again.  Calls that share a scratch must not overlap on the GPU.
 *   scatter_table / scatter_index as for mvb_sample.
 * Accumulation is fp32 in the tensor cores' order, which is not cuBLAS's: a logit can round to the neighbouring
 * bf16 value, so the token may differ from the unfused path where the two best logits are within one bf16 step.
 */
size_t mvb_lm_head_argmax_scratch_bytes(int max_rows);
int mvb_lm_head_argmax(const void* hidden_states, int64_t x_row_stride, const void* weight, int64_t w_row_stride,
                       int num_rows, int hidden, int vocab, int64_t* out, int64_t* scatter_table,
                       const int32_t* scatter_index, void* scratch, size_t scratch_bytes, int32_t* dev_status,
                       void* stream);

/*
 * Decoder-layer glue around the attention path.  A decode step of a small model is bound by the number
 * of kernels it launches, so the elementwise chains the models run between their GEMMs are fused.
 *
 * mvb_act_mul: out[t, i] = act(gate_up[t, i]) * gate_up[t, intermediate + i] on a packed
 *   [rows, 2 * intermediate] projection; act = SiLU (minivllm/models/models/qwen3.py:117-121) or
 *   tanh-GELU (gelu_tanh != 0, minivllm/models/models/gemma3.py:122-128).  The activation is rounded
 *   to bf16 before the product, as the unfused sequence rounds it.
 * mvb_add_rmsnorm: the residual update and the next RMSNorm of a decoder layer in one pass over a row:
 *     y' = y                       (y_weight == NULL; qwen3.py:146-155)
 *     y' = rmsnorm(y, y_weight)    (Gemma's post-attention / post-feedforward norm, gemma3.py:157-170)
 *     x  = bf16(x + y')            (in place, x is [rows, hidden] contiguous)
 *     out = rmsnorm(x, weight)     (the following input / post-attention / pre-feedforward / final norm)
 *   rmsnorm(v, w) = v * rsqrt(mean(v^2) + eps) * w, or * (1 + w) when unit_offset != 0, in fp32.
 *   hidden must be a multiple of 8 and at most 8192.
 * mvb_add_rmsnorm_last_tokens: the same residual add and norm, but only for the LAST token of every sequence of
 *   a packed prefill batch, gathered by the kernel itself: output row r is computed from source row
 *   cu_seqlens_q[r + 1] - 1, which is the row the reference picks with last_indices = cu_seqlens_q[1:] - 1
 *   (minivllm/models/models/qwen3.py:215-217, gemma3.py:258-260) AFTER running the final norm over every token.
 *   x is read only (the residual stream is not needed after the final norm); out is [num_seqs, hidden].
 */
int mvb_add_rmsnorm_last_tokens(const void* x, const void* y, int64_t y_row_stride, const void* y_weight,
                                const void* weight, void* out, const int32_t* cu_seqlens_q, int num_seqs, int hidden,
                                float eps, int unit_offset, void* stream);
int mvb_act_mul(const void* gate_up, int64_t in_row_stride, void* out, int64_t out_row_stride, int rows,
                int intermediate, int gelu_tanh, void* stream);
int mvb_add_rmsnorm(void* x, const void* y, int64_t y_row_stride, const void* y_weight, const void* weight,
                    void* out, int rows, int hidden, float eps, int unit_offset, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MINI_VLLM_B200_H_ */
