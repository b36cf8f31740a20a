/*
 * C ABI of libdsv4_prologue.so — the B200 (sm_100a) implementation of the
 * DeepSeek-V4 attention prologue and of the reader of the cache rows it writes.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless the
 * parameter name ends in `_host`.  No entry point allocates, synchronises or
 * reads device memory back unless its comment says so; work is enqueued on
 * `cuda_stream` (a cudaStream_t passed as void*, NULL = the legacy default
 * stream) of the CURRENT device.
 *
 * Return value of every int-returning function: 0 on success, a negative
 * DSV4_ERR_* code when the arguments are rejected before anything is launched,
 * or a positive cudaError_t reported by the launch.
 */
#ifndef DSV4_PROLOGUE_H
#define DSV4_PROLOGUE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV4_OK 0
#define DSV4_ERR_NULL_POINTER (-1) /* a required pointer is NULL */
#define DSV4_ERR_BAD_SIZE (-2)     /* negative size, num_tokens_insert > num_tokens, block too small */
#define DSV4_ERR_MISALIGNED (-3)   /* a pointer or stride is not aligned as the entry point requires */
#define DSV4_ERR_BAD_VARIANT (-4)  /* unknown kernel variant id */
#define DSV4_ERR_TOO_LARGE (-5)    /* size exceeds what the entry point supports */

/* Layout constants of one cached token (reference:
 * src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:35-43). */
#define DSV4_HEAD_DIM 512
#define DSV4_ROPE_DIM 64
#define DSV4_NOPE_DIM 448
#define DSV4_TOKEN_DATA_BYTES 576 /* 448 e4m3 + 64 bf16 */
#define DSV4_SCALE_BYTES 8        /* 7 UE8M0 codes + 1 zero byte */

/* Kernel variants selectable with dsv4_set_variant (0 = choose by problem size). */
#define DSV4_VARIANT_AUTO 0
#define DSV4_VARIANT_ROWS 1 /* one launch, 16-byte vector loads/stores through registers */
#define DSV4_VARIANT_BULK 2 /* persistent CTAs, bulk-async (TMA) copies through a shared-memory ring */

/*
 * The fused prologue.  Replaces the reference's Python+Triton operator
 *   fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(q, kv, k_cache, slot_mapping,
 *       position_ids, cos_sin_cache, eps, cache_block_size)
 * (src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:289-351,
 * kernel :20-286) with the same effects:
 *   q              bf16 [num_tokens, num_heads, 512], contiguous, rewritten in place:
 *                  weight-less RMSNorm over 512 (fp32, eps) then GPT-J RoPE on [448,512)
 *   kv             bf16 [num_tokens, 512], contiguous, read only
 *   k_cache        bytes; block b starts at k_cache + b*kv_block_stride_bytes and holds
 *                  cache_block_size*576 data bytes then cache_block_size*8 scale bytes
 *   slot_mapping   int64 [num_tokens_insert], num_tokens_insert <= num_tokens; token t is
 *                  stored at slot_mapping[t] unless that is negative or t >= num_tokens_insert
 *   position_ids   int64 [num_tokens]; row index into cos_sin_cache
 *   cos_sin_cache  fp32 [max_pos, 64] = 32 cos | 32 sin
 * Nothing is bounds-checked on the device (as in the reference): slots and positions
 * must be in range.  With q, kv and cos_sin_cache on 16-byte boundaries the vectorised kernels run; q and kv on any
 * 2-byte and cos_sin_cache on any 4-byte boundary (contiguous views that start inside their storage, which the
 * reference accepts) run on a kernel with 2-byte accesses and the same results.  k_cache may have any alignment
 * (a slower byte-store path is taken unless base and stride are multiples of 16).
 */
int dsv4_qnorm_rope_kv_insert(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping,
                              const int64_t* position_ids, const float* cos_sin_cache, float eps,
                              int64_t num_tokens, int64_t num_heads, int64_t num_tokens_insert,
                              int64_t cache_block_size, int64_t kv_block_stride_bytes, void* cuda_stream);

/*
 * Out-of-place form with head padding: q [num_tokens, num_heads, 512] is read only, the normalised and
 * rotated rows go to q_out [num_tokens, padded_heads, 512] (padded_heads >= num_heads, 16-byte aligned) and
 * heads num_heads..padded_heads-1 of every token are zero-filled; the KV side is identical.  This is how
 * vLLM >= 0.22 calls the operator (torch.ops._C.<same name> with an extra padded_heads argument, returning
 * the padded tensor); the reference pins the 8-argument in-place form (OP:289-298), so this entry point has
 * no counterpart there.  One launch, DSV4_VARIANT_ROWS kernel.
 */
int dsv4_qnorm_rope_kv_insert_padded(const void* q, void* q_out, const void* kv, void* k_cache, const int64_t* slot_mapping,
                                     const int64_t* position_ids, const float* cos_sin_cache, float eps, int64_t num_tokens,
                                     int64_t num_heads, int64_t padded_heads, int64_t num_tokens_insert,
                                     int64_t cache_block_size, int64_t kv_block_stride_bytes, void* cuda_stream);

/*
 * Same operator with the device-side range checks the reference lacks: a token whose
 * position is outside [0, max_pos) or whose slot is >= num_blocks*cache_block_size is
 * left unprocessed and a bit is OR-ed into *status (device int32, caller-zeroed):
 * bit 0 = bad position, bit 1 = bad slot.  Used by the test-suite in place of a
 * memory checker.  Always the DSV4_VARIANT_ROWS kernel.  No counterpart in the reference
 * (its kernel trusts its indices).
 */
int dsv4_qnorm_rope_kv_insert_checked(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping,
                                      const int64_t* position_ids, const float* cos_sin_cache, float eps,
                                      int64_t num_tokens, int64_t num_heads, int64_t num_tokens_insert,
                                      int64_t cache_block_size, int64_t kv_block_stride_bytes,
                                      int64_t num_blocks, int64_t max_pos, int32_t* status, void* cuda_stream);

/*
 * Reader of the rows written above: out[i, 0:512] (bf16, row stride out_row_stride
 * elements) = token stored at slots[i]: 448 values e4m3 * 2^(code-127) rounded to bf16,
 * then the 64 cached bf16 RoPE values; a negative slot gives a zero row.  The per-token
 * arithmetic of the reference's
 *   dequantize_and_gather_k_cache
 * (src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:86-120)
 * addressed by slot instead of (request, block table).
 */
int dsv4_gather_dequant_k_cache(const void* k_cache, const int64_t* slots, int64_t num_slots, void* out,
                                int64_t out_row_stride, int64_t cache_block_size,
                                int64_t kv_block_stride_bytes, void* cuda_stream);

/*
 * The reference operator
 *   dequantize_and_gather_k_cache(out, k_cache, seq_lens, gather_lens, block_table, block_size, offset,
 *                                 rope_dim, nope_dim, scale_slots)
 * (src/flaggems_vllm/ops/deepseek_v4_attention_dequantize_and_gather_k_cache.py:123-172, kernel :38-120):
 * for request r and i < gather_lens[r] (all of seq_lens[r] when gather_lens is NULL),
 *   out[r, offset + i, 0 : nope_dim + rope_dim]
 * is the cached token at position seq_lens[r] - gather_lens[r] + i, located through
 * block_table[r, position / cache_block_size]; nope_dim e4m3 values times 2^(code - 127) per group of 64,
 * rounded to bf16, then rope_dim cached bf16 values.  A cached token is nope_dim + 2*rope_dim data bytes;
 * a block holds cache_block_size of them, then cache_block_size * scale_slots scale bytes.
 * out is bf16 with element strides out_stride0 / out_stride1 and unit stride in the last dimension;
 * out_tokens (its second extent) only sizes the grid.  seq_lens, gather_lens and block_table
 * ([num_reqs, max_blocks_per_seq], contiguous) are int32, or int64 when index_is_int64 != 0.
 * num_reqs <= 65535.  The DeepSeek-V4 layout (448 / 64 / 8) with 16-byte aligned rows takes a
 * vectorised path; anything else a scalar one.
 */
int dsv4_dequantize_and_gather_k_cache(void* out, int64_t out_stride0, int64_t out_stride1, int64_t out_tokens,
                                       const void* k_cache, const void* seq_lens, const void* gather_lens,
                                       const void* block_table, int64_t num_reqs, int64_t max_blocks_per_seq,
                                       int64_t cache_block_size, int64_t kv_block_stride_bytes, int64_t offset,
                                       int32_t nope_dim, int32_t rope_dim, int32_t scale_slots, int32_t index_is_int64,
                                       void* cuda_stream);

/*
 * The step before the prologue.  Replaces the reference operator
 *   fused_q_kv_rmsnorm(qr, kv, q_weight, kv_weight, eps) -> (qr_out, kv_out)
 * (src/flaggems_vllm/ops/deepseek_v4_attention_fused_q_kv_rmsnorm.py:65-103, kernel :24-62):
 * out = (x * rsqrt(mean(x^2) + eps)) * weight per row, fp32 arithmetic, for the q low-rank
 * activations [num_tokens, q_size] and the latent KV [num_tokens, kv_size] in one launch.  All six
 * tensors bf16 with unit stride in the last dimension; row strides in elements; outputs are
 * caller-allocated.  Rows of up to 2048 elements with 16-byte aligned bases and strides stay in
 * registers (one read, one write); others take a two-pass scalar path.
 */
int dsv4_fused_q_kv_rmsnorm(const void* qr, void* qr_out, const void* q_weight, int64_t q_in_stride,
                            int64_t q_out_stride, int64_t q_size, const void* kv, void* kv_out, const void* kv_weight,
                            int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size, int64_t num_tokens, float eps,
                            void* cuda_stream);

/*
 * The same operator for the element types the reference kernel accepts besides bf16 (it loads rows and weights as fp32
 * whatever their type and stores in the row's type, :50-62 there): *_dtype 0 = bf16, 1 = fp16, 2 = fp32, given
 * separately for the q rows (input and output share it), the kv rows and the two weight vectors.  All bf16 is forwarded
 * to dsv4_fused_q_kv_rmsnorm; anything else runs one warp per row, two passes, element by element.
 */
int dsv4_fused_q_kv_rmsnorm_dtypes(const void* qr, void* qr_out, const void* q_weight, int64_t q_in_stride, int64_t q_out_stride,
                                   int64_t q_size, int32_t q_dtype, int32_t q_weight_dtype, const void* kv, void* kv_out,
                                   const void* kv_weight, int64_t kv_in_stride, int64_t kv_out_stride, int64_t kv_size,
                                   int32_t kv_dtype, int32_t kv_weight_dtype, int64_t num_tokens, float eps, void* cuda_stream);

/*
 * The attention epilogue that mirrors the prologue.  Replaces the reference operator
 *   fused_inv_rope_fp8_quant(o, positions, cos_sin_cache, n_groups, heads_per_group, nope_dim=448,
 *                            rope_dim=64, quant_group_size=128, eps, dtype, tma_aligned_scales)
 * (src/flaggems_vllm/ops/fused_inv_rope_fp8_quant.py:155-256, kernel :37-152) for head_dim 512 = 448 + 64
 * and groups of 128: inverse GPT-J RoPE on o[..., 448:512] (rounded to bf16, as the reference's torch
 * statement tests/test_fused_inv_rope_fp8_quant.py:150-198 does), then per group of 128 values
 * scale = max(amax, eps)/448 (power of two >= that when packed_ue8m0_scales) and e4m3(x / scale).
 *   o          bf16 [num_tokens, n_groups*heads_per_group, 512], element strides given, 16-byte aligned rows
 *   positions  int64 [num_tokens]; cos_sin_cache fp32 rows of 64 (32 cos | 32 sin), row stride in elements
 *   fp8_out    e4m3 bytes, contiguous [n_groups, num_tokens, heads_per_group*512]
 *   scale_out  element (g, t, k) at g*scale_stride_group + t + k*padded_tokens (4-byte elements):
 *              fp32 with k < heads_per_group*4, or int32 with k < heads_per_group holding the head's four
 *              UE8M0 exponent bytes (group j in byte j); columns t in [num_tokens, padded_tokens) are zeroed.
 *              padded_tokens = num_tokens rounded up to a multiple of 4.
 */
int dsv4_fused_inv_rope_fp8_quant(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                  const float* cos_sin_cache, int64_t cos_sin_stride, void* fp8_out, void* scale_out,
                                  int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int64_t n_groups,
                                  int64_t heads_per_group, float eps, int32_t packed_ue8m0_scales, void* cuda_stream);

/*
 * The same operator for every geometry the reference wrapper accepts (:193-200 there): head_dim = nope_dim + rope_dim a
 * multiple of quant_group_size, nope_dim % quant_group_size == quant_group_size - rope_dim (the rotary tail ends the last
 * group), rope_dim even; in addition quant_group_size must be even.  Same tensors and layouts with 512 replaced by
 * head_dim, 64 by rope_dim and 4 by head_dim / quant_group_size scale columns per head; o needs 2-byte alignment only.
 * packed_ue8m0_scales requires four groups per head (one int32 per head is the only packed layout in which the
 * reference's kernel and allocation agree).  448 / 64 / 128 with 16-byte aligned rows is forwarded to
 * dsv4_fused_inv_rope_fp8_quant; anything else runs one warp per (token, head), group by group, with IEEE divisions.
 */
int dsv4_fused_inv_rope_fp8_quant_geometry(const void* o, int64_t o_stride_token, int64_t o_stride_head, const int64_t* positions,
                                           const float* cos_sin_cache, int64_t cos_sin_stride, void* fp8_out, void* scale_out,
                                           int64_t scale_stride_group, int64_t num_tokens, int64_t padded_tokens, int64_t n_groups,
                                           int64_t heads_per_group, int64_t nope_dim, int64_t rope_dim, int64_t quant_group_size,
                                           float eps, int32_t packed_ue8m0_scales, void* cuda_stream);

/*
 * The sparse-indexer sibling of the prologue's KV insert.  Replaces the reference operator
 *   indexer_k_quant_and_cache(k, kv_cache, slot_mapping, quant_block_size, scale_fmt)
 * (src/flaggems_vllm/ops/indexer_k_quant_and_cache.py:103-132, kernel :44-100): token t of k
 * [num_tokens, head_dim] (bf16, or fp16 when k_is_fp16) goes to slot_mapping[t] (skipped when negative):
 * per group of quant_block_size values scale = max(amax, 1e-4)/448 (rounded up to a power of two when
 * scale_is_ue8m0), bytes = e4m3(x / scale).  Cache block b at b*cache_block_stride_bytes holds
 * cache_block_size*head_dim value bytes, then cache_block_size*(head_dim/quant_block_size) fp32 scales.
 */
int dsv4_indexer_k_quant_and_cache(const void* k, int64_t k_row_stride, int32_t k_is_fp16, void* kv_cache,
                                   int64_t cache_block_stride_bytes, const int64_t* slot_mapping, int64_t num_tokens,
                                   int64_t cache_block_size, int64_t head_dim, int64_t quant_block_size,
                                   int32_t scale_is_ue8m0, void* cuda_stream);

/*
 * The reader of the sparse-indexer key cache.  Replaces the reference operator
 *   cp_gather_indexer_k_quant_cache(k_cache, k_fp8, k_fp8_scale, block_table, cu_seqlen)
 * (src/flaggems_vllm/ops/cp_gather_indexer_k_quant_cache.py:129-190, kernel :24-126): output token t belongs to
 * the request b with cu_seqlen[b] <= t < cu_seqlen[b+1] (int32 [batch+1], non-decreasing; tokens outside every
 * request are left untouched); with o = t - cu_seqlen[b] its head_dim value bytes and num_quant_blocks fp32
 * scales are copied from cache block block_table[b*block_table_stride + o / cache_block_size] (int32), position
 * o % cache_block_size, to k_out + t*k_out_stride_bytes and scale_out + t*scale_out_stride_bytes.  Cache blocks
 * are laid out as for dsv4_indexer_k_quant_and_cache.
 */
int dsv4_cp_gather_indexer_k_quant_cache(const void* k_cache, int64_t cache_block_stride_bytes, void* k_out,
                                         int64_t k_out_stride_bytes, void* scale_out, int64_t scale_out_stride_bytes,
                                         const int32_t* block_table, int64_t block_table_stride, const int32_t* cu_seqlen,
                                         int64_t batch, int64_t num_tokens, int64_t cache_block_size, int64_t head_dim,
                                         int64_t num_quant_blocks, void* cuda_stream);

/*
 * Top-k positions inside a request -> slots of the paged cache.  Replaces the reference operator
 *   compute_global_topk_indices_and_lens(topk_indices, token_to_req_indices, block_table, block_size, is_valid_token)
 * (src/flaggems_vllm/ops/deepseek_v4_attention_compute_global_topk_indices_and_lens.py:128-161, kernel :49-125):
 * for token t and column i, p = topk_indices[t*topk_stride + i] (int32); global_indices[t*global_stride + i] =
 * block_table[token_to_req[t]*block_table_stride + p / block_size] * block_size + p % block_size, or -1 when
 * p < 0; lens[t] = number of non-negative entries of the row, 0 when is_valid_token[t] == 0 (is_valid_token may
 * be NULL: every token valid).  Strides in elements.
 */
int dsv4_compute_global_topk_indices_and_lens(const int32_t* topk_indices, int64_t topk_stride, const int32_t* token_to_req,
                                              const int32_t* block_table, int64_t block_table_stride, const int32_t* is_valid_token,
                                              int32_t* global_indices, int64_t global_stride, int32_t* lens, int64_t num_tokens,
                                              int64_t topk, int64_t block_size, void* cuda_stream);

/*
 * Rows of indices into the gathered key buffer for sparse prefill.  Replaces the reference operator
 *   combine_topk_swa_indices(topk_indices, query_start_loc, seq_lens, gather_lens, window_size, compress_ratio, topk, M, N)
 * (src/flaggems_vllm/ops/deepseek_v4_attention_combine_topk_swa_indices.py:109-161, kernel :30-106): query token t of
 * request b (query_start_loc[b] - query_start_loc[0] <= t < query_start_loc[b+1] - query_start_loc[0]) sits at position
 * pos = seq_lens[b] - query_len + (t - start); its row of combined_width int32 holds
 *   topk_len = min((pos+1)/compress_ratio, topk) entries topk_indices[t, i] + M*b, then
 *   swa_len = min(pos+1, window_size) entries M*b + N + j + pos - swa_len + 1 - (seq_lens[b] - gather_lens[b]),
 *   then -1 up to combined_width; lens[t] = topk_len + swa_len.  Rows of tokens no request covers are not written.
 * Requires topk <= topk_width and topk + window_size <= combined_width.  Strides in elements.
 */
int dsv4_combine_topk_swa_indices(const int32_t* topk_indices, int64_t topk_stride, int64_t topk_width,
                                  const int32_t* query_start_loc, const int32_t* seq_lens, const int32_t* gather_lens,
                                  int32_t* combined, int64_t combined_stride, int64_t combined_width, int32_t* lens,
                                  int64_t num_reqs, int64_t num_tokens, int64_t window_size, int64_t compress_ratio, int64_t topk,
                                  int64_t M, int64_t N, void* cuda_stream);

/*
 * Top-k selection of the sparse indexer.  Replace the reference operators
 *   top_k_per_row_decode(logits, next_n, seq_lens, indices, num_rows, stride0, stride1, top_k)
 *   top_k_per_row_prefill(logits, row_starts, row_ends, indices, num_rows, stride0, stride1, top_k)
 * (src/flaggems_vllm/ops/top_k_per_row_decode.py:1263-1399, src/flaggems_vllm/ops/top_k_per_row_prefill.py, wrapper
 * `top_k_per_row_prefill`): for row i of logits (fp32 [num_rows, vocab], element strides) and its range
 * [start, end) - decode: start = 0, end = seq_lens[i / next_n] - next_n + i % next_n + 1; prefill: row_starts[i],
 * row_ends[i]; both clipped to [0, vocab] - indices[i*top_k + j], j < k = min(top_k, end - start), are the positions
 * relative to start of the k largest values in any order (ties broken arbitrarily), the remaining entries are -1.
 * row_starts may be NULL (every range starts at 0), which is the call shape of the reference's
 *   persistent_topk(logits, lengths, output, workspace, k, max_seq_len)
 * (src/flaggems_vllm/ops/persistent_topk.py:2179-2342) with row_ends = lengths; its workspace is not needed here: the
 * kernel keeps its state in shared memory.
 * The selection orders values by their bit patterns: a NaN with the sign bit clear ranks above +inf, one with the
 * sign bit set below -inf.
 */
int dsv4_top_k_per_row_decode(const float* logits, int64_t stride0, int64_t stride1, int64_t next_n, const int32_t* seq_lens,
                              int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k, void* cuda_stream);
int dsv4_top_k_per_row_prefill(const float* logits, int64_t stride0, int64_t stride1, const int32_t* row_starts,
                               const int32_t* row_ends, int32_t* indices, int64_t num_rows, int64_t vocab, int64_t top_k,
                               void* cuda_stream);

/*
 * The activation quantiser in front of the FP8 projections.  Replaces the reference operator
 *   per_token_group_quant_fp8(x, group_size, eps, dtype, column_major_scales, scale_ue8m0)
 * (src/flaggems_vllm/ops/per_token_group_quant_fp8.py:226-330, kernels :25-215) for bf16 x [num_rows, num_cols]
 * (row stride in elements, unit inner stride) and e4m3fn output (contiguous [num_rows, num_cols] bytes): per group of
 * group_size consecutive values scale = max(amax, eps) * (1/448), made 2^ceil(log2(scale)) when scale_is_ue8m0, and
 * bytes = e4m3(x / scale).  The fp32 scale of (row, group) goes to scales[row*scale_stride_row +
 * group*scale_stride_group] (row-major [num_rows, num_cols/group_size]: strides (num_cols/group_size, 1); the
 * reference's column-major layout: (1, num_rows)).
 */
int dsv4_per_token_group_quant_fp8(const void* x, int64_t x_row_stride, void* out, float* scales, int64_t scale_stride_row,
                                   int64_t scale_stride_group, int64_t num_rows, int64_t num_cols, int64_t group_size, float eps,
                                   int32_t scale_is_ue8m0, void* cuda_stream);

/*
 * Block-wise activation quantisation, DeepSeek's `act_quant`.  Replaces the reference operator
 *   act_quant_triton(x, block_size, scale_fmt)
 * (src/flaggems_vllm/ops/act_quant.py:113-175, kernel :46-110): as dsv4_per_token_group_quant_fp8 with row-major scales
 * [num_rows, num_cols/block_size], except that the maximum is clamped at 1e-4 in fp32 and the bytes are
 * e4m3(x * (1/scale)); round_scale (scale_fmt is not None) makes the scale 2^ceil(log2(scale)).
 */
int dsv4_act_quant(const void* x, int64_t x_row_stride, void* out, float* scales, int64_t num_rows, int64_t num_cols, int64_t block_size,
                   int32_t round_scale, void* cuda_stream);

/*
 * The sparse-indexer prologue.  Replaces the reference operator
 *   fused_indexer_q_rope_quant(positions, index_q, index_q_cos_sin_cache, index_weights,
 *                              index_weights_softmax_scale, index_weights_head_scale, use_fp4)
 * (src/flaggems_vllm/ops/fused_indexer_q_rope_quant.py:283-410, kernels :69-280): GPT-J RoPE on the last
 * rot_dim values of each head of index_q (bf16 [T, H, head_dim], element strides), result rounded to bf16, then
 *   use_fp4 == 0: q_out = e4m3(x / s) bytes [T, H, head_dim] with s = 2^ceil(log2(max(amax_head, 1e-4)/448));
 *                 weights_out = weights * s * softmax_scale * head_scale
 *   use_fp4 != 0: per 32 values s = 2^ceil(log2(max(amax, 6*2^-126)/6)); q_out = e2m1(x / s) packed two per
 *                 byte (even index in the low nibble) [T, H, head_dim/2]; q_scales_out = exponent bytes
 *                 [T, H, head_dim/32]; weights_out = weights * softmax_scale * head_scale
 * Output strides in bytes.  cos_sin_cache rows = rot_dim/2 cosines then rot_dim/2 sines, fp32 or bf16.
 * weights [T, H] of dtype code 0 bf16 / 1 fp16 / 2 fp32; weights_out fp32.  head_dim 64, 128 or 256.
 */
int dsv4_fused_indexer_q_rope_quant(const int64_t* positions, const void* index_q, int64_t q_stride0, int64_t q_stride1,
                                    const void* cos_sin_cache, int64_t cos_sin_stride, int32_t cos_sin_is_bf16, int64_t rot_dim,
                                    void* q_out, int64_t out_stride0, int64_t out_stride1, void* q_scales_out,
                                    int64_t scale_stride0, int64_t scale_stride1, const void* weights, int64_t weights_stride,
                                    int32_t weights_dtype, float* weights_out, int64_t weights_out_stride, float softmax_scale,
                                    float head_scale, int64_t num_tokens, int64_t num_heads, int64_t head_dim, int32_t use_fp4,
                                    void* cuda_stream);

/*
 * Reads into *value_host, and clears, the error word the kernels of the current device keep:
 * bit 0 = a bounded wait inside the DSV4_VARIANT_BULK kernel ran out (its result is then
 * incomplete).  Synchronises the device.  0 after every healthy run.  No counterpart in the reference.
 */
int dsv4_device_error(int32_t* value_host);

/* The remaining entry points are housekeeping of this library and have no counterpart in the reference.
 *
 * Process-wide kernel variant (DSV4_VARIANT_*); also read once from the environment
 * variable DSV4_VARIANT.  Returns the previous value or DSV4_ERR_BAD_VARIANT. */
int dsv4_set_variant(int variant);
int dsv4_get_variant(void);

/* DSV4_VARIANT_BULK only.  Every wait of that kernel on a shared-memory barrier is bounded: after `cycles` SM cycles
 * (default 2e8, about 0.1 s; values above 2e9 are clamped, values <= 0 only read the setting) the waiting role gives up,
 * bit 0 of the device error word is set, the CTA's other roles leave their loops, the loader waits - bounded again - for
 * the copies it has issued, and the kernel returns with q and the cache partly processed.  The entry points still
 * return 0 in that case (the launch itself succeeded): a caller that selects the bulk variant must read
 * dsv4_device_error at its next synchronisation point.  Returns the previous limit. */
int64_t dsv4_set_bulk_wait_cycles(int64_t cycles);

/* Self-test of that give-up path, for test suites; not an operator.  Same arguments and effects as
 * dsv4_qnorm_rope_kv_insert on the bulk variant, except that the loader of tile `short_tile` (tiles are 16 rows:
 * first ceil(num_tokens_insert / 16) tiles of kv rows, then the tiles of q rows) announces 16 bytes it never sends,
 * so the waits on that tile's stage run out after the limit set with dsv4_set_bulk_wait_cycles.  Nothing traps and
 * nothing waits without a limit: the kernel returns by itself, dsv4_device_error then reads 1, and the rows of the
 * affected CTA from that tile on are left unprocessed. */
int dsv4_bulk_wait_selftest(void* q, const void* kv, void* k_cache, const int64_t* slot_mapping, const int64_t* position_ids,
                            const float* cos_sin_cache, float eps, int64_t num_tokens, int64_t num_heads,
                            int64_t num_tokens_insert, int64_t cache_block_size, int64_t kv_block_stride_bytes,
                            int64_t short_tile, void* cuda_stream);

/* Programmatic dependent launch for dsv4_qnorm_rope_kv_insert (rows variant; also read once from the environment
 * variable DSV4_PDL).  In modes 1 and 2 the kernel is launched so that it may start while the
 * preceding kernel of the stream is still finishing, and lets the kernel after it do the same once its own loads are
 * out, which hides most of the gap between back-to-back launches of decode-sized batches (256 tokens x 128 heads on
 * B200: 12.1 us per call against 14.3 us).
 *   mode 0: an ordinary launch.
 *   mode 2 (default): ordinary stream semantics - the kernel reads nothing before the preceding kernel has finished
 *           and its writes are visible; only the launch itself overlaps.
 *   mode 1: the kernel also fetches position_ids, slot_mapping and the cos/sin rows at once and waits for the
 *           preceding kernel only before it touches q, kv and the cache.  The caller promises that position_ids,
 *           slot_mapping and cos_sin_cache are not written by the kernel that precedes the call in the stream.
 * Returns the previous mode. */
int dsv4_set_pdl(int mode);

/* Where the rows variant of dsv4_qnorm_rope_kv_insert takes the cos/sin rows from (also read once from the environment
 * variable DSV4_TABLE_STAGING): -1 (default) = by launch size, 0 = every warp fetches the table row of its own q rows
 * into registers (no barrier; the choice for decode-sized launches), 1 = once per CTA through shared memory (less L2
 * traffic; the choice for large launches).  Results do not depend on it.  Returns the previous mode. */
int dsv4_set_table_staging(int mode);

/* Number of kernels this library has launched in this process (all entry points). */
int64_t dsv4_launch_count(void);

/* Human-readable text for a return code of this library. */
const char* dsv4_error_string(int code);

/* "dsv4-prologue <version> sm_100a". */
const char* dsv4_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DSV4_PROLOGUE_H */
