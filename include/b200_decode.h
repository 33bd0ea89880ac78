/*
 * b200_decode.h - C ABI of the B200 (sm_100a) decode hot path.
 *
 * One shared library, libb200decode.so.  Plain pointers and sizes only; every
 * pointer is a DEVICE pointer unless stated otherwise; `stream` is a
 * cudaStream_t passed as void*.  Unless an entry point says otherwise it
 *   - allocates nothing and frees nothing (the caller owns every buffer,
 *     including workspaces),
 *   - never synchronises the stream or the device,
 *   - returns 0 on success or a negative code (see b200_strerror); argument
 *     errors are detected on the host before anything is launched,
 *   - reports problems found on the device (a block id outside the pool, a
 *     bounded barrier wait that ran out, ...) by writing a positive code into
 *     the 4-byte status word at the start of the workspace it was given; the
 *     word is sticky (first error wins) and must be zero before first use.
 *     Read it with b200_read_status().
 *
 * The reference (AdvayMonga/inference-server) has no native interface: its
 * decode step is TorchBackend.decode_step_batched
 * (src/inference_server/backends/torch_backend.py:305-322), which hands dense
 * tensors to a HuggingFace model.  Each entry point below names the piece of
 * that step it replaces.
 */
#ifndef B200_DECODE_H_
#define B200_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes for the attention / KV entry points */
#define B200_DTYPE_BF16 0
#define B200_DTYPE_F32 1

/* ---------------------------------------------------------------- status -- */

int b200_abi_version(void);
/* Text for a return code (negative) or a device status word (positive). */
const char* b200_strerror(int code);
/* Thread-local detail string of the last failing call on this thread. */
const char* b200_last_error_detail(void);
/* Copies the device status word to the host and returns it negated (0 = clean).
 * The only entry point that synchronises `stream`. */
int b200_read_status(const void* status_word, void* stream);

/* ------------------------------------------------------- paged attention -- */

/*
 * Replaces: page gather kv_cache/hf_format.py:21-45 (blocks_to_dynamic_cache),
 * left-padded batch build backends/torch_backend.py:237-258, and the attention
 * arithmetic of the model forward called at torch_backend.py:314-320
 * (softmax(q K^T * scale) V per row with GQA head sharing, softmax in fp32).
 *
 *   q            [batch, num_q_heads, head_dim]
 *   k_pool/v_pool[num_blocks, num_kv_heads, page_size, head_dim] - the layout
 *                of kv_cache/block_manager.py:33-49, read in place
 *   block_table  [batch, max_pages_per_seq] int32 page ids (Block.block_id,
 *                kv_cache/block.py:18); all pages full except the last
 *   ctx_lens     [batch] int32 tokens to attend to (including this step's)
 *   out          [batch, num_q_heads, head_dim], same dtype as q
 *   workspace    b200_paged_attn_workspace_bytes(...) bytes; starts with the
 *                status word, then the per-split partial results.  Calls
 *                sharing a workspace must not overlap on the GPU.
 *   split_tokens tokens per split of the KV length, a multiple of 16
 *
 * bf16 pools with page_size 16, head_dim 64 or 128 and at most 16 q heads per
 * kv head and 1, 2, 4 or 8 kv heads take the TMA split-K kernel; anything else (fp32, other pages or head
 * sizes up to 256) takes a plain fp32-arithmetic kernel without a split.
 */
size_t b200_paged_attn_workspace_bytes(int batch, int num_q_heads, int head_dim,
                                       int max_pages_per_seq, int page_size, int split_tokens);
int b200_paged_attn_decode(const void* q, const void* k_pool, const void* v_pool,
                           const int32_t* block_table, const int32_t* ctx_lens, void* out,
                           void* workspace, size_t workspace_bytes, int batch, int num_q_heads,
                           int num_kv_heads, int head_dim, int page_size, int num_blocks,
                           int max_pages_per_seq, float scale, int split_tokens, int dtype,
                           void* stream);

/*
 * b200_paged_attn_decode for the rows of a prompt chunk: batch rows 2i and 2i+1 are two consecutive tokens of
 * one sequence and SHARE block_table row 2i (row 2i+1 of the table is not read); ctx_lens stays per row (the
 * causal mask: token t attends to t+1 positions).  The second row rides in the upper half of the m16 MMA tile,
 * which up to 8 query heads per kv head leave idle, so every page is fetched once for two rows.  Same results,
 * bit for bit, as b200_paged_attn_decode on the same rows.  bf16, page_size 16, head_dim 128 with 4 kv heads or
 * head_dim 64 with 2, at most 8 query heads per kv head; workspace as for b200_paged_attn_decode.  Replaces,
 * for cache-hit prompts, the page gather of kv_cache/hf_format.py:21-45 + the HF prompt attention.
 */
int b200_paged_attn_decode_pairs(const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_table, const int32_t* ctx_lens, void* out,
                                 void* workspace, size_t workspace_bytes, int batch, int num_q_heads,
                                 int num_kv_heads, int head_dim, int page_size, int num_blocks,
                                 int max_pages_per_seq, float scale, int split_tokens, void* stream);

/*
 * Replaces, for a prompt or the uncached suffix of one: the page gather of a cached prefix into a dense
 * cache (kv_cache/hf_format.py:21-45) and the causally masked prompt attention inside the model forward
 * (torch_backend.py:107-147; chunked prefill: scheduler.py:312-353).  A chunk of num_tokens consecutive
 * prompt tokens of ONE sequence, at positions first_position .., whose K/V are already in their page slots,
 * attends to the sequence's pages in place; the row of position p sees tokens 0..p.  One CTA covers 128 rows
 * of the score matrix (128 / group consecutive positions x the group's query heads), so a page is fetched once
 * per 128 rows; no split over the context, no workspace.
 *
 *   q, out            [num_tokens, num_q_heads, head_dim] bf16
 *   block_table_row   [max_pages_per_seq] int32: the sequence's pages
 *   status_word       optional device int32 for device-side findings (bad block id, position past the table)
 * bf16, page_size 16; head_dim 128 with 8 or 16 query heads per kv head, or head_dim 64 with 4.
 * head_dim 128 (q and out 16-byte aligned) runs on the tcgen05 tensor cores with the scores and the output
 * accumulated in TMEM; the other shapes, and every shape when the environment variable B200_PREFILL_MMA_SYNC is
 * set to a non-zero value, on the mma.sync kernel.
 */
int b200_paged_attn_prefill(const void* q, const void* k_pool, const void* v_pool,
                            const int32_t* block_table_row, void* out, void* status_word, int num_tokens,
                            int first_position, int num_q_heads, int num_kv_heads, int head_dim,
                            int page_size, int num_blocks, int max_pages_per_seq, float scale, void* stream);

/*
 * Paged decode attention for callers that cannot allocate device memory.
 * No counterpart in the reference: it exists for hosts of this library that own
 * no allocator at the point of the call - a server whose device memory was
 * carved up at start-up and is fully handed out, a plugin that is only lent its
 * input and output buffers, or code that runs while a CUDA graph is being
 * captured, where cudaMalloc is not permitted.
 *
 * Same arithmetic and the same kernels as b200_paged_attn_decode for bf16 pools
 * with page_size 16, head_dim 64 or 128 and 1, 2, 4 or 8 kv heads (other shapes
 * are refused: use b200_paged_attn_decode).  The per-split partial results go to
 * a fixed B200_STATIC_SCRATCH_BYTES array inside the library image instead of a
 * caller workspace; every GPU that loads the library holds that array until the
 * process exits.  The call is refused with a "workspace too small" error when
 *   batch * num_q_heads * ceil(max_pages_per_seq * 16 / split_tokens)
 *         * (head_dim * 4 + 8)  bytes (the (m, l) block rounded up to 256)
 * exceed it.  The function itself calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *
 *   status_word  caller-owned 4-byte device word for device-side error codes,
 *                zero before first use, or NULL.
 *
 * The first call on each device looks up the device address of the array
 * (cudaGetSymbolAddress, with that device current) and keeps it; make that
 * first call before starting any stream capture.  Nothing in the array has to
 * start at zero and nothing is cleared: every call overwrites the slots it later
 * reads.  All calls on one device share the array, so two calls whose kernels may
 * overlap on the GPU (different streams without an ordering between them) race
 * on it; order them, or give one of them a workspace of its own through
 * b200_paged_attn_decode.
 */
#define B200_STATIC_SCRATCH_BYTES (32u << 20)
int b200_paged_attn_decode_static(const void* q, const void* k_pool, const void* v_pool,
                                  const int32_t* block_table, const int32_t* ctx_lens, void* out,
                                  void* status_word, int batch, int num_q_heads, int num_kv_heads,
                                  int head_dim, int page_size, int num_blocks, int max_pages_per_seq,
                                  float scale, int split_tokens, void* stream);

/*
 * Replaces: the per-step KV growth DynamicCache.update does with torch.cat
 * inside the forward called at torch_backend.py:314-320, and gives decode the
 * page write the reference only has for prompts
 * (kv_cache/cache_manager.py:185-214, _store_kv_in_blocks).
 *
 *   k_new/v_new  [batch, num_kv_heads, head_dim]
 *   positions    [batch] int32 token index the row is written at
 *   status_word  4-byte device word (may be NULL)
 */
int b200_kv_append(const void* k_new, const void* v_new, void* k_pool, void* v_pool,
                   const int32_t* block_table, const int32_t* positions, void* status_word,
                   int batch, int num_kv_heads, int head_dim, int page_size, int num_blocks,
                   int max_pages_per_seq, int dtype, void* stream);

/* ----------------------------------------------------- dense projections -- */

/*
 * Replaces: the bf16 linear layers of the model forward called at torch_backend.py:314-320 (transformers
 * Qwen3MoeAttention q/k/v/o projections, the router's gate projection, lm_head), which the reference runs as
 * library GEMMs.  y[m, n] = sum_k x[m, k] * w[n, k] with fp32 accumulation on the tensor cores (tcgen05).
 * The weight tile is the M side of the MMA and the step's rows the N side, so a decode batch streams the
 * weights once; with few weight tiles K is split over the CTAs of a thread-block cluster, whose fp32 partial
 * tiles meet in the workspace and are summed in rank order (deterministic, no atomics).
 *
 *   x [num_rows, in_features] bf16,  w [out_features, in_features] bf16 (the checkpoint layout),
 *   y [num_rows, out_features] bf16, 8-byte aligned.  in_features must be a multiple of 64; x and w 16-byte
 *   aligned.
 *   workspace  b200_dense_gemm_workspace_bytes(num_rows, out_features) bytes, 16-byte aligned, or NULL: the
 *              product is then computed without a K split (slower when there are few weight tiles)
 *   k_split    0 = chosen by the library; 1, 2, 4 or 8 = CTAs that share one weight tile
 *   status_word  optional device int32 for a bounded wait that ran out
 */
size_t b200_dense_gemm_workspace_bytes(int num_rows, int out_features);
int b200_dense_gemm_bf16(const void* x, const void* w, void* y, void* workspace, size_t workspace_bytes,
                         void* status_word, int num_rows, int out_features, int in_features, int k_split,
                         void* stream);

/*
 * Replaces, in one kernel: the fused q/k/v projection of an attention block and what follows it before the
 * attention itself - per-head RMSNorm of q and k, rotary embedding, and the write of this step's K and V into
 * their page slots (transformers Qwen3MoeAttention.forward up to the attention call, with the decode-time form of
 * the page write at kv_cache/cache_manager.py:185-214): b200_dense_gemm_bf16 with the work of
 * b200_qk_norm_rope_append in its epilogue.  A weight tile is one head (head_dim 128); the tile's bf16 result is
 * normalised, rotated and stored from shared memory, so the [rows, heads, 128] projection output never goes to
 * global memory.  Same results, bit for bit, as the two separate calls (the projection without a K split).
 *
 *   x [num_rows, in_features] bf16; wqkv [(Hq + 2 Hkv) * 128, in_features] bf16: q heads, k heads, v heads
 *   other arguments as b200_qk_norm_rope_append
 */
int b200_qkv_rope_append_supported(int head_dim, int in_features);
int b200_qkv_rope_append_gemm(const void* x, const void* wqkv, const void* q_norm_weight,
                              const void* k_norm_weight, const void* cos_table, const void* sin_table,
                              const int32_t* positions, const int32_t* block_table, void* q_out, void* k_pool,
                              void* v_pool, void* status_word, int num_rows, int num_q_heads, int num_kv_heads,
                              int head_dim, int in_features, float eps, int page_size, int num_blocks,
                              int max_pages_per_seq, int max_positions, void* stream);

/*
 * Replaces: lm_head followed by the argmax over the vocabulary (torch_backend.py:314-321:
 * `outputs.logits[:, -1, :].argmax(dim=-1)`).  The same GEMM with a running arg-max per row kept in registers
 * across the vocabulary tiles; the [num_rows, vocab] logits are never written.  The largest fp32 logit wins,
 * equal logits go to the lower token id.
 *
 *   x [num_rows, hidden] bf16 (final-normed hidden states), w [vocab_size, hidden] bf16,
 *   next_tokens [num_rows] int64.  num_rows <= 256 per call; hidden a multiple of 64.
 *   workspace  b200_lm_head_argmax_workspace_bytes() bytes, 16-byte aligned (per-CTA candidates)
 */
size_t b200_lm_head_argmax_workspace_bytes(void);
int b200_lm_head_argmax(const void* x, const void* w, int64_t* next_tokens, void* workspace,
                        size_t workspace_bytes, void* status_word, int num_rows, int vocab_size,
                        int hidden, void* stream);

/* ----------------------------------------------------- fused step glue -- */

/*
 * Replaces: the residual add and RMSNorm ops of the decoder layer inside the
 * forward called at torch_backend.py:314-320 (statistics in fp32, eps inside the
 * square root, normalised value rounded to bf16 before the weight multiply).
 *
 *   x       [num_rows, hidden] bf16 residual stream; updated in place to
 *           x + delta when delta is not NULL
 *   delta   [num_rows, hidden] bf16 or NULL
 *   out     [num_rows, hidden] bf16 = weight * normalise(x)
 */
int b200_add_rmsnorm(void* x, const void* delta, const void* weight, float eps, int num_rows,
                     int hidden, void* out, void* stream);

/*
 * Replaces: per-head q/k RMSNorm, rotary embedding (rotate-half) and the KV
 * cache growth of the attention module under the same forward, writing k and v
 * straight into their page slot (kv_cache/cache_manager.py:185-214 for prompts).
 *
 *   qkv        [batch, num_q_heads + 2*num_kv_heads, head_dim] bf16: q heads,
 *              then k heads, then v heads
 *   cos/sin    [max_positions, head_dim] bf16 tables
 *   positions  [batch] int32 index of this step's token
 *   q_out      [batch, num_q_heads, head_dim] bf16
 */
int b200_qk_norm_rope_append(const void* qkv, const void* q_norm_weight, const void* k_norm_weight,
                             const void* cos_table, const void* sin_table,
                             const int32_t* positions, const int32_t* block_table, void* q_out,
                             void* k_pool, void* v_pool, void* status_word, int batch,
                             int num_q_heads, int num_kv_heads, int head_dim, float eps,
                             int page_size, int num_blocks, int max_pages_per_seq,
                             int max_positions, void* stream);

/*
 * Replaces, in one kernel: the residual add and post-attention RMSNorm of the decoder layer, the router's
 * linear layer (`gate`) and Qwen3MoeTopKRouter (fp32 softmax, top-k, renormalisation) of the forward called at
 * torch_backend.py:314-320 - b200_add_rmsnorm, the router projection and b200_moe_route back to back, with the
 * router logits kept on the chip in fp32.  A cluster of 8 CTAs owns 16 rows; each CTA takes an eighth of the
 * hidden dimension and the partial sums of squares and partial logits meet through distributed shared memory,
 * summed in rank order.
 *
 *   x [num_rows, hidden] bf16, updated in place to x + delta when delta is not NULL
 *   normed_out [num_rows, hidden] bf16 = norm_weight * normalise(x)   (the MoE layer's input)
 *   router_weight [num_experts, hidden] bf16
 *   topk_ids / topk_weights  as b200_moe_route (num_valid_rows: see there)
 *   logits_out  optional [num_rows, num_experts] fp32
 * hidden a multiple of 512, num_experts a multiple of 16 and at most 128: b200_add_rmsnorm_route_supported.
 */
int b200_add_rmsnorm_route_supported(int hidden, int num_experts, int top_k);
int b200_add_rmsnorm_route(void* x, const void* delta, const void* norm_weight, float eps,
                           const void* router_weight, int num_rows, int hidden, int num_experts, int top_k,
                           int renormalize, const int32_t* num_valid_rows, void* normed_out, int32_t* topk_ids,
                           float* topk_weights, float* logits_out, void* stream);

/* ------------------------------------------------------------------- MoE -- */

/*
 * Replaces: the router of the sparse MoE block run by the forward at
 * torch_backend.py:314-320 (fp32 softmax over experts, top-k, optional
 * renormalisation).  Ties between equal logits go to the lower expert id.
 *
 *   logits       [num_tokens, num_experts], logits_dtype B200_DTYPE_F32 or
 *                B200_DTYPE_BF16 (the router projection's own output type)
 *   num_valid_rows  optional device int32: rows at or beyond it are padding of a
 *                fixed-shape step and get expert id -1 ("no expert") and weight 0;
 *                b200_moe_permute* leave such pairs out (row_of_pair -1) and the
 *                combine kernels add nothing for them.  NULL: every row is real.
 *   topk_ids     [num_tokens, top_k] int32, value-descending
 *   topk_weights [num_tokens, top_k] fp32
 */
int b200_moe_route(const void* logits, int logits_dtype, int num_tokens, int num_experts, int top_k,
                   int renormalize, const int32_t* num_valid_rows, int32_t* topk_ids, float* topk_weights,
                   void* stream);

/*
 * Replaces: the sort-by-expert / offsets step of the grouped expert forward
 * under the same call.  Pairs (token, slot) are numbered token * top_k + slot
 * and stably sorted by expert id.
 *
 *   sorted_pair_ids [num_tokens * top_k] pair id held by each sorted row
 *   row_of_pair     [num_tokens * top_k] sorted row of each pair (inverse)
 *   expert_offsets  [num_experts + 1] first sorted row of each expert
 *   tiles           b200_moe_max_tiles(...) * 16 bytes, {expert,row0,rows,0}
 *                   int32 records of <=128 rows, or NULL (then num_tiles NULL)
 *   num_tiles       1 int32
 *   workspace       b200_moe_permute_workspace_bytes(...); starts with the
 *                   status word
 */
size_t b200_moe_permute_workspace_bytes(int num_tokens, int num_experts, int top_k);
int b200_moe_max_tiles(int num_tokens, int num_experts, int top_k);
int b200_moe_permute(const int32_t* topk_ids, int num_tokens, int num_experts, int top_k,
                     int32_t* sorted_pair_ids, int32_t* row_of_pair, int32_t* expert_offsets,
                     void* tiles, int32_t* num_tiles, int tile_experts, void* workspace,
                     size_t workspace_bytes, void* stream);
/* tile_experts: only experts [0, tile_experts) get row tiles (0 = all).  The expert-parallel receive side
 * sorts its slots with one extra dummy expert for empty slots and sets tile_experts to the real count. */

/*
 * b200_moe_permute and b200_act_quant_fp8 (below) in one pass: the token rows of
 * x [num_tokens, hidden] bf16 are quantised and written straight to their sorted
 * rows of xq / x_scale.  Same outputs, one kernel fewer on the step's critical path.
 */
int b200_moe_permute_quant(const int32_t* topk_ids, const void* x, int num_tokens, int num_experts,
                           int top_k, int hidden, int32_t* sorted_pair_ids, int32_t* row_of_pair,
                           int32_t* expert_offsets, void* tiles, int32_t* num_tiles, void* xq,
                           float* x_scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Expert-parallel form of b200_moe_permute_quant (no counterpart in the reference, which is single-device):
 * experts are owned by ep_world ranks in equal contiguous id ranges.  The quantised row of pair p goes to row
 * slot_of_pair[p] = owner * ep_capacity + (position among this rank's rows for that owner) of the send buffers
 * xq_send / x_scale_send [ep_world * ep_capacity rows], expert_of_slot gets the owner-local expert id of every
 * used slot and the "empty" id num_experts / ep_world of every unused one, pairs beyond the capacity get
 * slot -1 and set *overflow to 1.
 */
int b200_moe_permute_quant_ep(const int32_t* topk_ids, const void* x, int num_tokens, int num_experts,
                              int top_k, int hidden, int ep_world, int ep_capacity,
                              int32_t* sorted_pair_ids, int32_t* row_of_pair, int32_t* expert_offsets,
                              void* tiles, int32_t* num_tiles, void* xq_send, float* x_scale_send,
                              int32_t* slot_of_pair, int32_t* expert_of_slot, int32_t* overflow,
                              void* workspace, size_t workspace_bytes, void* stream);

/* dst row i = src row order[i], for e4m3 rows [rows, hidden] and their scales [rows, hidden/128]
 * (the receive side of the expert-parallel exchange brings its slots into expert-sorted order with it). */
int b200_gather_rows_fp8(const void* src_q, const float* src_scale, const int32_t* order, int num_rows,
                         int hidden, void* dst_q, float* dst_scale, void* stream);

/*
 * Replaces: the dynamic per-token activation quantisation of the FP8 expert
 * layers (one fp32 scale per row per 128 columns: s = amax / 448, 1 for an
 * all-zero group; q = e4m3(x / s)).
 *
 *   x            [num_tokens, hidden] bf16
 *   row_of_pair  NULL: row t is written to row t.  Otherwise [num_tokens*top_k]:
 *                row t is written to each of its top_k sorted rows.
 *   xq           [rows, hidden] e4m3 bytes;  x_scale [rows, hidden / 128] fp32
 */
int b200_act_quant_fp8(const void* x, const int32_t* row_of_pair, int num_tokens, int hidden,
                       int top_k, void* xq, float* x_scale, void* stream);

/*
 * Replace: the expert matmuls of the forward at torch_backend.py:314-320 on
 * e4m3 weights with fp32 128x128 block scales (tcgen05 grouped GEMM).
 *
 * gate_up: h = silu(W13[e][:inter] x) * (W13[e][inter:] x) per sorted row,
 *          re-quantised per row per 128 columns.
 *   xq [num_rows, hidden] e4m3, x_scale [num_rows, hidden/128]
 *   w13 [num_experts, 2*inter, hidden] e4m3,
 *   w13_scale_inv [num_experts, 2*inter/128, hidden/128] fp32
 *   hq [num_rows, inter] e4m3, h_scale [num_rows, inter/128] fp32
 * down:    y = W2[e] h per sorted row.
 *   w2 [num_experts, hidden, inter] e4m3,
 *   w2_scale_inv [num_experts, hidden/128, inter/128] fp32
 *   y_sorted [num_rows, hidden] bf16; with out_row_map (int32 [num_rows], may be NULL) sorted row r is
 *   written to row out_row_map[r] instead of row r
 * tiles/num_tiles come from b200_moe_permute; status_word may be NULL.
 *
 * weight_layout: B200_WEIGHTS_ROW_MAJOR - the arrays above as written (the
 * reference checkpoint layout); B200_WEIGHTS_TILED - the same e4m3 values
 * re-ordered at load time into contiguous 128x128 blocks,
 * [num_experts, rows/128, cols/128, 128, 128], so that every TMA box of W is
 * one sequential 16 KiB read.  Scales are the same in both.
 */
#define B200_WEIGHTS_ROW_MAJOR 0
#define B200_WEIGHTS_TILED 1
int b200_moe_fp8_gemm_gate_up(const void* xq, const float* x_scale, const void* w13,
                              const float* w13_scale_inv, const void* tiles,
                              const int32_t* num_tiles, void* hq, float* h_scale,
                              void* status_word, int num_rows, int num_experts, int hidden,
                              int inter, int weight_layout, void* stream);
int b200_moe_fp8_gemm_down(const void* hq, const float* h_scale, const void* w2,
                           const float* w2_scale_inv, const void* tiles, const int32_t* num_tiles,
                           void* y_sorted, const int32_t* out_row_map, void* status_word, int num_rows,
                           int num_experts,
                           int hidden, int inter, int weight_layout, void* stream);

/*
 * Replaces: the routing-weight multiply and per-token sum over the top_k expert
 * outputs.  out[t] = sum_k topk_weights[t,k] * y_sorted[row_of_pair[t,k]] in
 * fp32, k ascending, rounded to bf16.  A negative row_of_pair entry (a pair
 * the expert-parallel dispatch had to drop) contributes nothing.
 */
int b200_moe_combine(const void* y_sorted, const int32_t* row_of_pair, const float* topk_weights,
                     int num_tokens, int hidden, int top_k, void* out, void* stream);

/*
 * b200_moe_combine followed by b200_add_rmsnorm in one kernel: the combined
 * expert output is rounded to bf16, added to the residual stream x (in place)
 * and the result is normalised with `weight` into `out`.
 */
int b200_moe_combine_add_rmsnorm(const void* y_sorted, const int32_t* row_of_pair,
                                 const float* topk_weights, void* x, const void* weight, float eps,
                                 int num_tokens, int hidden, int top_k, void* out, void* stream);

/*
 * The whole FP8 MoE layer for one batch of tokens: route, permute, quantise,
 * gate/up GEMM, down GEMM, combine, in that order on `stream`.
 *
 *   x [num_tokens, hidden] bf16, router_logits [num_tokens, num_experts] of
 *   logits_dtype, out [num_tokens, hidden] bf16, workspace
 *   b200_moe_fp8_workspace_bytes(...) bytes, 256-byte aligned, zero before first use.
 *
 * The _add_rmsnorm form ends with b200_moe_combine_add_rmsnorm instead of
 * b200_moe_combine: `residual` [num_tokens, hidden] is updated in place and
 * `normed_out` receives norm_weight * rmsnorm(residual) - the input of the next
 * decoder layer.
 */
size_t b200_moe_fp8_workspace_bytes(int num_tokens, int num_experts, int top_k, int hidden,
                                    int inter);
int b200_moe_fp8_forward(const void* x, const void* router_logits, int logits_dtype, const void* w13,
                         const float* w13_scale_inv, const void* w2, const float* w2_scale_inv,
                         void* out, void* workspace, size_t workspace_bytes, int num_tokens,
                         int num_experts, int top_k, int hidden, int inter, int renormalize,
                         int weight_layout, void* stream);
int b200_moe_fp8_forward_add_rmsnorm(const void* x, const void* router_logits, int logits_dtype,
                                     const void* w13, const float* w13_scale_inv, const void* w2,
                                     const float* w2_scale_inv, void* residual,
                                     const void* norm_weight, float eps, void* normed_out,
                                     void* workspace, size_t workspace_bytes, int num_tokens,
                                     int num_experts, int top_k, int hidden, int inter,
                                     int renormalize, int weight_layout, void* stream);

/*
 * The _add_rmsnorm form for tokens that are already routed (b200_add_rmsnorm_route, or the model's own
 * router as the experts module of transformers is called: `experts(hidden_states, top_k_index,
 * top_k_weights)`): permute+quantise, the two grouped GEMMs, combine + residual + norm.
 *   topk_ids [num_tokens, top_k] int32 (-1 = no expert), topk_weights [num_tokens, top_k] fp32
 */
int b200_moe_fp8_routed_add_rmsnorm(const void* x, const int32_t* topk_ids, const float* topk_weights,
                                    const void* w13, const float* w13_scale_inv, const void* w2,
                                    const float* w2_scale_inv, void* residual, const void* norm_weight,
                                    float eps, void* normed_out, void* workspace, size_t workspace_bytes,
                                    int num_tokens, int num_experts, int top_k, int hidden, int inter,
                                    int weight_layout, void* stream);

/*
 * ---------------------------------------------------------------------------
 * Expert parallelism over peer memory.  None of this has a counterpart in the
 * reference, which is single-device; it serves the multi-GPU partition of the
 * MoE layer (experts owned by ep_world <= 8 ranks in equal contiguous id ranges).
 *
 * Every rank keeps its receive buffers in one device allocation that the other
 * ranks of the node map (b200_ipc_*), so that the dispatch and the return path
 * store rows straight into the owner's memory over NVLink:
 *
 *   xq_recv  [ep_world * ep_capacity, hidden] e4m3     row s * ep_capacity + i =
 *   xs_recv  [ep_world * ep_capacity, hidden/128] f32  the i-th row rank s sent here
 *   id_recv  [ep_world * ep_capacity] int32            its local expert id, or
 *                                                      num_experts / ep_world if empty
 *   y_recv   [ep_world * ep_capacity, hidden] bf16     row d * ep_capacity + i = the
 *                                                      expert output of the i-th row this
 *                                                      rank sent to rank d
 *   flags    [8] int32 per exchange phase, zero before first use
 *
 * The *_peers arguments are host arrays of ep_world device pointers, entry r =
 * that buffer of rank r as mapped in this process (entry ep_rank = this rank's own).
 * ---------------------------------------------------------------------------
 */

/* b200_moe_permute_quant_ep with the rows, scales and expert ids written into the owners' xq_recv / xs_recv /
 * id_recv (row ep_rank * ep_capacity + position) instead of local send buffers.  slot_of_pair as above. */
int b200_moe_permute_quant_ep_p2p(const int32_t* topk_ids, const void* x, int num_tokens, int num_experts,
                                  int top_k, int hidden, int ep_world, int ep_capacity, int ep_rank,
                                  int32_t* sorted_pair_ids, int32_t* row_of_pair, int32_t* expert_offsets,
                                  void* tiles, int32_t* num_tiles, void* const* xq_peers,
                                  void* const* xs_peers, void* const* id_peers, int32_t* slot_of_pair,
                                  int32_t* overflow, void* workspace, size_t workspace_bytes, void* stream);

/* b200_moe_fp8_gemm_down whose epilogue returns every row to the rank it came from: with
 * o = out_row_map[r] (the receive slot of sorted row r), the row is written to row
 * ep_rank * ep_capacity + o % ep_capacity of y_recv of rank o / ep_capacity. */
int b200_moe_fp8_gemm_down_p2p(const void* hq, const float* h_scale, const void* w2,
                               const float* w2_scale_inv, const void* tiles, const int32_t* num_tiles,
                               void* const* y_peers, const int32_t* out_row_map, void* status_word,
                               int num_rows, int num_experts, int hidden, int inter, int weight_layout,
                               int ep_world, int ep_capacity, int ep_rank, void* stream);

/* Receive side of the exchange in one call: b200_moe_permute over the received expert ids (one per row, experts
 * [tile_experts, num_experts) are ranked but get no tiles and no copy - the dummy expert of empty slots) fused
 * with b200_gather_rows_fp8 of the rows into that order.  num_experts <= 256.  Workspace:
 * b200_moe_permute_workspace_bytes(num_rows, num_experts, 1). */
int b200_moe_permute_gather_fp8(const int32_t* ids, int num_rows, int num_experts, int tile_experts,
                                const void* src_q, const float* src_scale, int hidden, int32_t* sorted_ids,
                                int32_t* row_of_id, int32_t* expert_offsets, void* tiles, int32_t* num_tiles,
                                void* dst_q, float* dst_scale, void* workspace, size_t workspace_bytes,
                                void* stream);

/*
 * Flag exchange that orders one rank's peer stores before another rank's reads.  epoch is a device int32
 * owned by this rank (one per phase, zero before first use); flag_peers[r] is the flags array of that phase
 * on rank r.  signal: epoch += 1 and flags[ep_rank] of every rank = epoch (after all earlier work of the
 * stream).  wait: returns when every entry of this rank's flags has reached its epoch; the wait is bounded
 * (about a second), after which the status word gets a peer-timeout code and the stream carries on.
 * barrier = signal + wait in one launch.  All ranks must issue the same sequence of phases.
 * status_word (may be NULL) must head an int32 array of at least 64 words: word 0 is the sticky status, words
 * 16..23 accumulate (modulo 2^32) the nanoseconds this rank has spent waiting for rank 0..7 - a diagnostic
 * for load imbalance between the ranks.
 */
int b200_ep_signal(void* const* flag_peers, int32_t* epoch, int ep_rank, int ep_world, void* stream);
int b200_ep_wait(const int32_t* local_flags, const int32_t* epoch, int ep_world, void* status_word,
                 void* stream);
int b200_ep_barrier(void* const* flag_peers, int32_t* epoch, int ep_rank, int ep_world, void* status_word,
                    void* stream);

/*
 * CUDA IPC for the buffers above.  export: the 64-byte handle of the allocation that contains ptr, and ptr's
 * offset inside it.  import (in another process of the node, once per handle): maps the allocation with
 * peer access and returns its base (for b200_ipc_close) and base + offset.
 */
int b200_ipc_export(const void* ptr, void* handle_out_64_bytes, uint64_t* offset_out);
int b200_ipc_import(const void* handle_64_bytes, uint64_t offset, void** base_out, void** ptr_out);
int b200_ipc_close(void* base);

#ifdef __cplusplus
}
#endif
#endif /* B200_DECODE_H_ */
