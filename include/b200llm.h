/*
 * b200llm.h — C ABI of the B200 (sm_100a) kernels behind the continuous-batching
 * prefill/decode step of the nano-vLLM-style engine in ZenoAFfectionate/LLM_from_Scratch.
 *
 * The reference engine has no native layer: its attention layer (the part that would call a
 * store_kvcache kernel, a varlen prefill attention and a paged decode attention) is missing from
 * the repository.  What the reference does define is the contract those kernels must honour —
 * the metadata tensors built by engine/model_runner.py (prepare_prefill :202-249, prepare_decode
 * :253-278), the KV pool layout of allocate_kv_cache (:162-190) and the padding conventions of
 * the CUDA-graph replay (:295-310).  Every entry point below cites the part of that contract it
 * implements.
 *
 * Conventions
 *   - every pointer is a BORROWED device pointer unless its name ends in _host; the library never
 *     allocates, frees or retains memory;
 *   - `stream` is a cudaStream_t passed as void*; a call only enqueues work on that stream and
 *     never synchronises the host, so every call can be captured in a CUDA graph;
 *   - metadata dtypes are exactly the reference's: slot_mapping and context_lens int64,
 *     block_tables and cu_seqlens int32; -1 is legal padding in slot_mapping and block_tables;
 *   - calls are reentrant and take no locks.  The only process-wide state is a few per-device caches (SM count,
 *     "shared-memory limit raised" flags, the address of the built-in scratch array) that are filled on first
 *     use without synchronisation: concurrent first calls from several host threads store identical values;
 *   - return value: 0 on success, a negative B200_ERR_* code for argument / launch errors that
 *     are detected on the host.  Faults detected on the device (a block id or slot outside the
 *     pool) never dereference the bad address: the access is skipped and a B200_ERR_* code is
 *     stored to `status` (a caller-owned device int32, may be NULL); read it with
 *     b200_read_status at the next host sync point;
 *   - dtype: B200_DTYPE_F32 or B200_DTYPE_BF16 is the element type of q/k/v/caches/outputs.
 *     Arithmetic is always accumulated in fp32.
 */
#ifndef B200LLM_H_
#define B200LLM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 9

#define B200_DTYPE_F32 0
#define B200_DTYPE_BF16 1

#define B200_OK 0
#define B200_ERR_ARG (-1)          /* null pointer, negative size, inconsistent head counts */
#define B200_ERR_ALIGN (-2)        /* pointer or stride not aligned as the kernel requires   */
#define B200_ERR_UNSUPPORTED (-3)  /* shape / dtype outside what the kernels implement       */
#define B200_ERR_LAUNCH (-4)       /* the CUDA runtime refused the launch                    */
#define B200_ERR_WORKSPACE (-5)    /* workspace smaller than *_workspace_bytes asks for      */
#define B200_ERR_BOUNDS (-6)       /* device-side: block id or slot outside the pool         */
#define B200_ERR_NO_DEVICE (-7)    /* no usable CUDA device                                  */
#define B200_ERR_TOO_LARGE (-8)    /* scratch needed exceeds a fixed built-in capacity       */
#define B200_ERR_TIMEOUT (-9)      /* device-side: a bounded barrier wait gave up            */

int b200_abi_version(void);
const char* b200_strerror(int code);

/* Number of SMs of the current device (148 on B200); <0 on error. */
int b200_sm_count(void);

/* Copies the device status word to the host (synchronises `stream`) and clears it. */
int b200_read_status(int32_t* status, int32_t* status_host, void* stream);

/* ---------------------------------------------------------------------------------------------
 * XXH64 of a byte string with seed 0, and the chained block hash built on it.
 * Replaces BlockManager.compute_hash (engine/block_manager.py:45-57), which calls the third-party
 * xxhash package: hash = XXH64( [8-byte little-endian prefix hash, if prefix != -1] ||
 * int32-little-endian token ids ).  Host-only; no GPU work.
 * ------------------------------------------------------------------------------------------- */
uint64_t b200_xxh64(const void* data_host, size_t len, uint64_t seed);
uint64_t b200_block_hash(const int32_t* token_ids_host, int32_t num_tokens, uint64_t prefix_hash,
                         int32_t has_prefix);
/* The whole chain at once: out_hashes[i] for every full block i of the token list (prefix of block 0:
 * none, of block i: out_hashes[i-1]).  Returns the number of full blocks, or -1 on a bad argument. */
int64_t b200_block_hash_chain(const int32_t* token_ids_host, int64_t num_tokens, int32_t block_size,
                              uint64_t* out_hashes);

/* ---------------------------------------------------------------------------------------------
 * The KV-block pool on the host, natively: BlockManager (engine/block_manager.py:8-157) as a handle.  Blocks are
 * handed out oldest-free-first (the reference's FIFO deque, :60-78); full blocks are sealed with the chained
 * hash above and found again by later prompts (:85-114) after a token-by-token comparison; reference counts
 * start at 1 (the reference starts at 0 and so leaks unshared blocks, :23-26; this is the engine's corrected
 * default mode), a released block keeps its contents and can be revived, and a hit never covers a whole
 * prompt.  Host-only, no GPU work; a handle is not thread-safe.
 *   b200_pool_allocate    blocks for a new sequence (allocate, :85-114): writes ceil(num_tokens/block_size) block
 *                         ids, *num_cached_out = tokens covered by reused blocks; returns the number of
 *                         blocks, or B200_ERR_TOO_LARGE when the pool runs dry (state partly applied, as
 *                         the reference's IndexError would leave it)
 *   b200_pool_deallocate  releases a table, last block first (deallocate, :116-127)
 *   b200_pool_append      decode-time growth (append, :136-157): see the definition's comment
 *   b200_pool_open_block / b200_pool_seal_block  the two halves of append for several decode steps per
 *                         scheduling decision: open ahead, seal once the tokens are known
 *   b200_pool_lookup      the block a chained hash currently resolves to, or -1
 *   b200_pool_snapshot    free ids oldest first (returns their number), reference counts, sealed flags, hashes
 * ------------------------------------------------------------------------------------------- */
void* b200_pool_create(int64_t num_blocks, int32_t block_size);
void b200_pool_destroy(void* pool);
int64_t b200_pool_num_free(const void* pool);
int64_t b200_pool_allocate(void* pool, const int32_t* token_ids_host, int64_t num_tokens, int32_t* table_out_host,
                           int64_t* num_cached_out_host);
int b200_pool_deallocate(void* pool, const int32_t* table_host, int64_t num_blocks);
int64_t b200_pool_append(void* pool, int32_t last_block, int32_t prev_block, int64_t num_tokens,
                         const int32_t* last_block_tokens_host);
int64_t b200_pool_open_block(void* pool);
int b200_pool_seal_block(void* pool, int32_t block, int32_t prev_block, const int32_t* block_tokens_host);
int64_t b200_pool_lookup(const void* pool, uint64_t hash);
int64_t b200_pool_snapshot(const void* pool, int32_t* free_order_host, int32_t* ref_counts_host,
                           uint8_t* sealed_host, uint64_t* hashes_host);

/* ---------------------------------------------------------------------------------------------
 * Step metadata on the host, natively (ModelRunner.prepare_prefill / prepare_decode, engine/model_runner.py:
 * 202-278), written straight into caller-owned (pinned) arrays.  Block tables arrive as one flat int32 array
 * with offsets: sequence i owns tables[table_offsets[i] : table_offsets[i + 1]].
 *   b200_prepare_prefill  the non-cached suffix of every sequence: cu_seqlens_q / cu_seqlens_k int32 [n + 1],
 *                         positions int64 [T] (num_cached + j for packed token j), slot_mapping int64 [T],
 *                         max_seqlens[0..1] = longest q / k; returns T (<= capacity) or a negative code
 *   b200_prepare_decode   one token per sequence: context_lens, slot_mapping int64 [n], block_tables int32
 *                         [n, width] padded with -1
 * ------------------------------------------------------------------------------------------- */
int64_t b200_prepare_prefill(int32_t num_seqs, const int64_t* num_tokens_host, const int64_t* num_cached_host,
                             const int64_t* table_offsets_host, const int32_t* tables_host, int32_t block_size,
                             int32_t* cu_seqlens_q_host, int32_t* cu_seqlens_k_host, int64_t* positions_host,
                             int64_t* slot_mapping_host, int64_t capacity, int32_t* max_seqlens_host);
int b200_prepare_decode(int32_t num_seqs, const int64_t* num_tokens_host, const int64_t* table_offsets_host,
                        const int32_t* tables_host, int32_t block_size, int64_t* context_lens_host,
                        int64_t* slot_mapping_host, int32_t* block_tables_host, int64_t width);

/* ---------------------------------------------------------------------------------------------
 * store_kvcache: k_cache[slot_mapping[t], :, :] = k[t, :, :] (same for v); slot < 0 is skipped.
 * Contract: engine/model_runner.py:184-190 (pool [num_blocks, block_size, Hkv, D] per layer, so a
 * slot is one row of [num_slots, Hkv*D]), :226-230 (prefill slots), :261 (decode slot) and
 * :300-301 (-1 padding under graph replay).
 *   k, v            [num_tokens, Hkv, D]; rows Hkv*D contiguous, token stride given in ELEMENTS
 *                   (k/v may be column slices of a fused qkv projection)
 *   k_cache,v_cache [num_slots, Hkv, D] contiguous
 *   v and v_cache may both be NULL for a single pool (the MLA latent cache: Hkv = 1,
 *   D = kv_lora_rank + rope_dim)
 * ------------------------------------------------------------------------------------------- */
int b200_store_kvcache(const void* k, const void* v, int64_t k_token_stride,
                       int64_t v_token_stride, void* k_cache, void* v_cache,
                       const int64_t* slot_mapping, int32_t num_tokens, int32_t num_kv_heads,
                       int32_t head_dim, int64_t num_slots, int32_t dtype, int32_t* status,
                       void* stream);

/* ---------------------------------------------------------------------------------------------
 * Paged GQA decode attention: one query token per sequence attends to its whole context through
 * block_tables.  Arithmetic = GroupedQueryAttention.forward cache branch
 * (model/attention/GQA.py:105-130) with the dense cache replaced by the paged pool; metadata =
 * prepare_decode (engine/model_runner.py:253-278).
 *   q, out        [batch, Hq, D] contiguous
 *   k_cache       [num_blocks, block_size, Hkv, D]
 *   block_tables  [batch, bt_stride] int32, entries beyond ceil(context_len/block_size) are
 *                 never read (-1 or stale values are fine)
 *   context_lens  [batch] int64, includes the token being decoded; <= 0 writes a zero row
 *   workspace     b200_paged_decode_gqa_workspace_bytes(...) bytes, 256-byte aligned; holds the arrival
 *                 counters and partial results of contexts split across thread blocks.  Its first
 *                 B200_DECODE_COUNTER_BYTES must be zero when the buffer is first used (one cudaMemset after
 *                 allocating it); every call leaves them zero again, whatever the shapes of successive calls.
 *                 The rest needs no initialisation.  Two calls that overlap on the GPU need two workspaces.
 * ------------------------------------------------------------------------------------------- */
#define B200_DECODE_COUNTER_BYTES ((size_t)256 << 10)
size_t b200_paged_decode_gqa_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                             int32_t num_kv_heads, int32_t head_dim,
                                             int32_t dtype);
int b200_paged_decode_gqa(const void* q, const void* k_cache, const void* v_cache, void* out,
                          const int32_t* block_tables, int64_t bt_stride,
                          const int64_t* context_lens, int32_t batch, int32_t num_q_heads,
                          int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                          int64_t num_blocks, float scale, void* workspace, size_t workspace_bytes,
                          int32_t dtype, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Paged GQA decode for callers that cannot allocate device memory (no counterpart in the
 * reference, whose engine allocates freely through torch).  Same arguments and results as
 * b200_paged_decode_gqa minus the workspace: the split-context scratch is a fixed
 * B200_STATIC_SCRATCH_BYTES (8 MiB) device array inside the library, held by every GPU that loads
 * the library until the process exits.  It is meant for hosts that gave all
 * device memory to the KV pool, or that may not call an allocator on the decode path.
 *   - calls no cudaMalloc/cudaFree or any allocating routine;
 *   - returns B200_ERR_TOO_LARGE when the call would take the split-context kernel (bf16, block_size 16,
 *     head_dim 32/64/128, 16-byte aligned q and caches) and b200_paged_decode_gqa_workspace_bytes(...) for
 *     the shape exceeds the capacity (nothing is launched); shapes served by the general kernel need no
 *     scratch and are never refused;
 *   - the first call on each device looks up the array's device address (a host-side symbol query,
 *     made with that device current); make that first call before starting any stream capture;
 *   - all calls share the array: calls that overlap on the GPU (two streams, two threads) race on
 *     it.  Nothing in it has to be cleared between calls (the counters at its head start at zero when the
 *     library is loaded and every call returns them to zero).
 * ------------------------------------------------------------------------------------------- */
#define B200_STATIC_SCRATCH_BYTES ((size_t)8 << 20)
int b200_paged_decode_gqa_static(const void* q, const void* k_cache, const void* v_cache,
                                 void* out, const int32_t* block_tables, int64_t bt_stride,
                                 const int64_t* context_lens, int32_t batch, int32_t num_q_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                                 int64_t num_blocks, float scale, int32_t dtype, int32_t* status,
                                 void* stream);

/* ---------------------------------------------------------------------------------------------
 * Ragged (varlen) causal prefill attention over sequences packed with cu_seqlens.
 * Arithmetic = scaled_dot_product_attention (model/attention/utils.py:51-63) per sequence with
 * the causal mask of TransformerLM.forward (model/transformer.py:174-176), bottom-right aligned
 * when seqlen_k > seqlen_q (GQA.py:108-113), KV heads shared as GQA.py:118-125; metadata =
 * prepare_prefill (engine/model_runner.py:202-249).
 *   q   [total_q, Hq, Dqk]   token stride q_token_stride (elements), heads contiguous
 *   k   [total_k, Hkv, Dqk], v [total_k, Hkv, Dv]: the new tokens' keys/values when
 *       block_tables == NULL (then cu_seqlens_k must equal cu_seqlens_q);
 *   when block_tables != NULL (some prefix is cached, model_runner.py:231-237) keys/values are
 *       read from k_cache/v_cache through block_tables [num_seqs, bt_stride] and k/v are ignored
 *       (the caller has already stored the new tokens with b200_store_kvcache);
 *   out [total_q, Hq, Dv] contiguous.
 *   total_q_tokens / total_k_tokens are the row counts of q and of k/v (>= cu_seqlens[num_seqs],
 *   which the host knows from its tensors): they bound the TMA tensor maps built over q/k/v.
 *   plan (may be NULL): a tile list written by b200_prefill_plan for the same cu_seqlens_q, with its
 *   tile_rows and capacity.  With a plan the tiled kernels launch one CTA per listed tile (longest
 *   first) instead of num_seqs x ceil(max_seqlen_q / tile) CTAs, and neither num_seqs nor max_seqlen_q
 *   shapes the grid any more, so a step with fixed buffer sizes can be captured in a CUDA graph:
 *   pass num_seqs = the capacity of cu_seqlens (unused trailing sequences have length 0).
 *   A plan whose tile_rows does not match the kernel chosen for the shape is ignored.
 *   slot_mapping (may be NULL): int64, one slot per new token (the rows of k / v; -1 = skip), as prepare_prefill
 *   builds it (model_runner.py:226-230).  When given, the call also performs the step's store_kvcache:
 *   k_cache[slot] = k row, v_cache[slot] = v row for the pool [num_blocks, block_size, Hkv, D] (k, v, k_cache,
 *   v_cache, block_size and num_blocks are then required, with or without block_tables, and head_dim_qk must
 *   equal head_dim_v).  The scatter is enqueued ahead of the attention grid inside this call, so keys read
 *   through block_tables include the new tokens.
 * ------------------------------------------------------------------------------------------- */
int b200_prefill_varlen(const void* q, const void* k, const void* v, void* out,
                        int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                        int64_t total_q_tokens, int64_t total_k_tokens,
                        const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                        int32_t num_seqs, int32_t max_seqlen_q, int32_t max_seqlen_k,
                        int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim_qk,
                        int32_t head_dim_v, float scale, const void* k_cache, const void* v_cache,
                        const int32_t* block_tables, int64_t bt_stride, int32_t block_size,
                        int64_t num_blocks, const int64_t* slot_mapping, const int32_t* plan,
                        int32_t plan_tile_rows, int32_t plan_capacity, int32_t dtype, int32_t* status,
                        void* stream);

/* The same attention for keys stored in two parts, as the expanded form of multi-head latent attention
 * has them (model/attention/MLA.py:93-95,131: k = [k_nope of the head | k_rope shared by all heads]):
 *   k_head [total_k, H, head_dim_qk - tail_dim]  per-head columns, token stride k_head_token_stride
 *   k_tail [total_k, tail_dim]                   last tail_dim columns of every head's key
 *   q      [total_q, H, head_dim_qk], v [total_k, H, head_dim_v], out [total_q, H, head_dim_v]
 * so the rotary part is never copied into every head.  Keys/values are packed (no paged prefix);
 * total_q_tokens / total_k_tokens are the row counts of q and of k_head / k_tail / v, as above.
 * bf16, (head_dim_qk, tail_dim, head_dim_v) = (192, 64, 128), all parts 16-byte aligned; anything else
 * returns B200_ERR_UNSUPPORTED (the caller then expands the keys and uses b200_prefill_varlen).  plan: as above, for the
 * tile_rows of b200_prefill_tile_rows(head_dim_qk, head_dim_v, H, H, dtype). */
int b200_prefill_varlen_shared_tail(const void* q, const void* k_head, const void* k_tail, const void* v,
                                    void* out, int64_t q_token_stride, int64_t k_head_token_stride,
                                    int64_t k_tail_token_stride, int64_t v_token_stride,
                                    int64_t total_q_tokens, int64_t total_k_tokens,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    int32_t num_seqs, int32_t max_seqlen_q, int32_t num_heads,
                                    int32_t head_dim_qk, int32_t tail_dim, int32_t head_dim_v, float scale,
                                    const int32_t* plan, int32_t plan_tile_rows, int32_t plan_capacity,
                                    int32_t dtype, int32_t* status, void* stream);

/* Tile list for b200_prefill_varlen, computed on the device from cu_seqlens_q (one small launch per
 * step; all layers of the step reuse it).
 *   b200_prefill_tile_rows: query rows per tile of the kernel that serves this shape with packed keys
 *     (256 or 128 tcgen05: head dims 128 / 192+128, and head_dim 64 with query heads in groups of four;
 *     64 mma.sync), or 0 when only the general kernel applies (no plan then).
 *   b200_prefill_plan_bytes: size of `plan` for up to total_q_tokens rows in up to num_seqs sequences;
 *     its capacity in tiles is bytes / 4 - 4.
 *   b200_prefill_plan: max_seqlen_q is a host-side upper bound of the longest sequence
 *     (more than 4096 tiles in one sequence: B200_ERR_UNSUPPORTED).  Layout: int32 header
 *     {tiles, tile_rows, capacity, 0}, then (sequence << 16 | tile) per tile, highest tiles first. */
int32_t b200_prefill_tile_rows(int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim_qk,
                               int32_t head_dim_v, int32_t dtype);
size_t b200_prefill_plan_bytes(int64_t total_q_tokens, int32_t num_seqs, int32_t tile_rows);
int b200_prefill_plan(const int32_t* cu_seqlens_q, int32_t num_seqs, int32_t max_seqlen_q,
                      int32_t tile_rows, int32_t* plan, size_t plan_bytes, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * MLA latent-cache decode (absorbed form).  Arithmetic = MultiHeadLatentAttention.forward cache
 * branch (model/attention/MLA.py:153-178) between the two weight einsums:
 *   score = (q_abs . c^T + q_rope . pe^T) * scale ; P = softmax(score) ; out_latent = P . c
 * with c/pe read from a paged latent pool whose rows are [kv_lora_rank | rope_dim].
 *   q_abs [batch, H, r], q_rope [batch, H, dr], out_latent [batch, H, r] contiguous
 *   latent_cache [num_blocks, block_size, r + dr]
 * ------------------------------------------------------------------------------------------- */
size_t b200_mla_decode_workspace_bytes(int32_t batch, int32_t num_heads, int32_t kv_lora_rank,
                                       int32_t rope_dim, int32_t dtype);
int b200_mla_decode(const void* q_abs, const void* q_rope, const void* latent_cache,
                    void* out_latent, const int32_t* block_tables, int64_t bt_stride,
                    const int64_t* context_lens, int32_t batch, int32_t num_heads,
                    int32_t kv_lora_rank, int32_t rope_dim, int32_t block_size,
                    int64_t num_blocks, float scale, void* workspace, size_t workspace_bytes,
                    int32_t dtype, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Residual-stream RMSNorm with the reference's optional fused residual add (model/utils.py:54-67):
 *   xf = float(x) [+ float(residual)];  y = (weight * xf * rsqrt(mean(xf^2) + eps)) in x's dtype;
 *   residual_out = xf in x's dtype (may be NULL).  x, y, residual_out: [num_rows, dim] contiguous in
 *   `dtype`; residual (may be NULL) in `residual_dtype`; weight fp32 [dim].
 * ------------------------------------------------------------------------------------------- */
int b200_add_rmsnorm(const void* x, const void* residual, const float* weight, void* y,
                     void* residual_out, int64_t num_rows, int32_t dim, float eps, int32_t dtype,
                     int32_t residual_dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Everything GroupedQueryAttention.forward does between its projections and the attention call
 * (model/attention/GQA.py:81-102), plus the store_kvcache scatter, in one pass over the fused
 * projection output qkv [num_tokens, >= (Hq + 2 Hkv) * D] (token stride in elements):
 *   q, k: RMSNorm over the whole projected vector (eps as given: the reference's layers have eps=None,
 *   which torch evaluates in fp32 with the fp32 machine epsilon when the weight is fp32), rounded to the
 *   dtype, then half-split RoPE (model/attention/utils.py:34-45) in fp32 at positions[t] using rope_table [rope_positions, D] = cat(cos, sin), rounded to the dtype;
 *   q_out [num_tokens, Hq, D], k_out [num_tokens, Hkv, D];
 *   if k_cache != NULL: k_cache[slot] = k_out row, v_cache[slot] = raw v row, slot < 0 skipped.
 * ------------------------------------------------------------------------------------------- */
int b200_qk_norm_rope_store(const void* qkv, int64_t qkv_token_stride, const float* q_norm_weight,
                            const float* k_norm_weight, const float* rope_table,
                            int64_t rope_positions, const int64_t* positions, void* q_out, void* k_out,
                            void* k_cache, void* v_cache, const int64_t* slot_mapping,
                            int64_t num_slots, int64_t num_tokens, int32_t num_q_heads,
                            int32_t num_kv_heads, int32_t head_dim, float eps, int32_t dtype,
                            int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Everything MultiHeadLatentAttention.forward does between its projections and the attention
 * (model/attention/MLA.py:114-131 and the cache write of :137-138), one pass per token:
 *   q_up    [num_tokens, >= H*head_dim + H*rope_dim] (row stride in elements): the fused q up-projection,
 *           q_nope of all heads followed by q_rope of all heads;
 *   kv_down [num_tokens, >= kv_lora_rank + rope_dim]: the kv down-projection followed by k_rope.
 *   q_out    [num_tokens, H, head_dim + rope_dim] = [ q_nope | RoPE(q_rope) ]
 *   rows_out [num_tokens, kv_lora_rank + rope_dim] = [ RMSNorm(c) * kv_norm_weight | RoPE(k_rope) ]
 *            (may be NULL); the same row is written to latent_cache[slot_mapping[t]] when
 *            latent_cache != NULL (slot < 0 skipped).
 * RoPE is half-split, fp32, and reads cos from rope_table[pos, 0 : rope_dim/2] and "sin" from
 * rope_table[pos, rope_dim/2 : rope_dim]: the reference slices a table built for head_dim to its first
 * rope_dim columns (model/attention/utils.py:38), which this reproduces.  bf16 only.
 * ------------------------------------------------------------------------------------------- */
int b200_mla_prologue(const void* q_up, int64_t q_up_stride, const void* kv_down, int64_t kv_down_stride,
                      const float* kv_norm_weight, const float* rope_table, int64_t rope_width,
                      int64_t rope_positions, const int64_t* positions, void* q_out, void* rows_out,
                      void* latent_cache, const int64_t* slot_mapping, int64_t num_slots,
                      int64_t num_tokens, int32_t num_heads, int32_t head_dim, int32_t rope_dim,
                      int32_t kv_lora_rank, float eps, int32_t dtype, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * MoE routing for inference (Gate.forward, model/architecture/moe.py:45-90, and the grouping by
 * expert that MOE.moe_infer does with argsort + bincount on the host, moe.py:297-307), on the device.
 *   gate_logits [num_tokens, num_experts] in `dtype` (= x @ gate_weight^T), expert_bias fp32.
 *   scores = sigmoid(logits); top_k experts by logits + bias (ties to the lower index); weights =
 *   selected scores / (their sum + 1e-10) when top_k > 1; all rounded as the dtype would.
 * Outputs, rows ordered by (expert, token):
 *   sorted_token / sorted_expert int32 [num_tokens*top_k], sorted_weight `dtype` [num_tokens*top_k],
 *   expert_offsets int32 [num_experts] (exclusive end of every expert's rows),
 *   slot_to_row int32 [num_tokens, top_k]: row of token t's j-th expert in ascending expert order.
 * identity_tail != 0: sorted_token has num_tokens*top_k + num_tokens entries and the last num_tokens are
 *   0, 1, 2, ...: one gather then also yields the rows of a shared expert (see b200_moe_grouped_gemm).
 * One launch for num_tokens <= 256, two (count, scatter) above; `workspace` of
 * b200_moe_route_workspace_bytes() bytes (0 for num_tokens <= 256) holds the per-CTA counts.
 * Limits: num_experts <= 64, top_k <= 8, num_tokens <= 65536 (else B200_ERR_UNSUPPORTED).
 * ------------------------------------------------------------------------------------------- */
size_t b200_moe_route_workspace_bytes(int32_t num_tokens, int32_t num_experts);
int b200_moe_route(const void* gate_logits, const float* expert_bias, int32_t num_tokens,
                   int32_t num_experts, int32_t top_k, int32_t* sorted_token, int32_t* sorted_expert,
                   void* sorted_weight, int32_t* expert_offsets, int32_t* slot_to_row,
                   int32_t identity_tail, void* workspace, size_t workspace_bytes, int32_t dtype,
                   void* stream);

/* The gate projection, the routing above and (optionally) the gather of the routed rows in ONE launch, for
 * batches of at most 256 tokens (decode): gate_logits = bf16(x . gate_weight^T) (Gate.forward, moe.py:49-52),
 * then exactly b200_moe_route.  x [num_tokens, d_model] bf16 contiguous, gate_weight [num_experts, d_model] bf16.
 * gathered (may be NULL): [num_tokens*top_k (+ num_tokens with identity_tail), d_model], row i = x[sorted_token[i]]
 * (the index_select that feeds b200_moe_grouped_gemm); one thread block copies the rows, so pass it for small
 * batches only.  workspace: b200_moe_gate_route_workspace_bytes() bytes, 256-byte aligned, zero when first
 * used (its first word is a ticket counter that every call returns to zero).  More than 256 tokens, another
 * dtype, d_model % 8 != 0 or a gate matrix above 160 KiB: B200_ERR_UNSUPPORTED (use a GEMM and b200_moe_route). */
size_t b200_moe_gate_route_workspace_bytes(void);
int b200_moe_gate_route(const void* x, const void* gate_weight, const float* expert_bias, int32_t num_tokens,
                        int32_t num_experts, int32_t top_k, int32_t d_model, int32_t* sorted_token,
                        int32_t* sorted_expert, void* sorted_weight, int32_t* expert_offsets,
                        int32_t* slot_to_row, int32_t identity_tail, void* gathered, void* workspace,
                        size_t workspace_bytes, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * SwiGLU of fused up-projection rows (model/architecture/mlp.py:61-67: w2(silu(w1 x) * w3 x)):
 *   h [num_rows, 2*d_ff] = [w1 x | w3 x];  act [num_rows, d_ff] = silu(h1 + b1) * (h3 + b3).
 * `bias` (may be NULL: already added by the GEMM) is [experts, 2*d_ff]; row r uses the bias row
 * row_expert[r] (row 0 when row_expert is NULL).  Bias add, silu and product are each rounded to the
 * dtype, like the tensor-op sequence they replace.
 * ------------------------------------------------------------------------------------------- */
int b200_swiglu(const void* h, const void* bias, const int32_t* row_expert, void* act, int64_t num_rows,
                int32_t d_ff, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * MoE combine (MOE.moe_infer, moe.py:312-339, and the shared expert, moe.py:272-273):
 *   out[t] = sum_j round(round(expert_out[row] + bias[row_expert[row]]) * row_weight[row]),
 *   row = slot_to_row[t, j], j ascending (= ascending expert id), every partial sum rounded to the
 *   dtype as the reference's scatter_add_ in the activation dtype does; then + shared[t] if given.
 * expert_out [num_tokens*top_k, d_model] in grouped (sorted) row order; bias [experts, d_model] or NULL.
 * ------------------------------------------------------------------------------------------- */
int b200_moe_combine(const void* expert_out, const void* bias, const int32_t* row_expert,
                     const void* row_weight, const int32_t* slot_to_row, const void* shared, void* out,
                     int64_t num_tokens, int32_t top_k, int32_t d_model, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Grouped GEMM over rows grouped by expert (the per-expert loop of MOE.moe_infer, moe.py:299-339),
 * bf16, fp32 accumulation on the tensor cores.  Expert e owns rows [offsets[e-1], offsets[e]) of
 * x [num_rows, k_dim] (expert_offsets as b200_moe_route writes them; read on the device).
 *   mode 0: out [num_rows, n_out] = x . W_e^T (+ bias[e] if given), w [experts, n_out, k_dim].
 *   mode 1: out [num_rows, n_out] = silu(x . W1_e^T + b1) * (x . W3_e^T + b3), n_out = d_ff,
 *           w [experts, 2*d_ff, k_dim] = rows of w1 then rows of w3, bias [experts, 2*d_ff] or NULL
 *           (mlp.py:61-67); GEMM result, bias add, silu and product are each rounded to bf16.
 * dense_rows > 0: the last dense_rows of the num_rows rows are not grouped: they all use weight set
 *   number num_experts (w and bias then hold num_experts + 1 sets) — a shared expert applied to every token
 *   (moe.py:272-273) computed by the same launch, in chunks that cost a CTA what an expert's rows cost.
 * mode | B200_MOE_GEMM_EARLY_LAUNCH: the launch is a programmatic dependent of the kernel before it in
 *   the stream: the prologue and the first ring of weight tiles overlap that kernel's tail, and only the
 *   reads of x wait for it.  The caller asserts that w, bias and expert_offsets were complete before
 *   that kernel started (they come from two or more launches back, as in route -> gather -> up -> down).
 * Requires k_dim % 8 == 0 and 16-byte aligned x, w (B200_ERR_ALIGN).  A wait that runs out inside
 * the kernel sets *status to B200_ERR_TIMEOUT.
 * ------------------------------------------------------------------------------------------- */
#define B200_MOE_GEMM_EARLY_LAUNCH 0x100
int b200_moe_grouped_gemm(const void* x, const void* w, const void* bias, void* out,
                          const int32_t* expert_offsets, int64_t num_rows, int32_t num_experts,
                          int32_t dense_rows, int32_t n_out, int32_t k_dim, int32_t mode, int32_t dtype,
                          int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode metadata of the next step, computed on the device from the step that just ran, so that several
 * decode steps can be launched back to back (host counterpart: ModelRunner.prepare_decode,
 * engine/model_runner.py:253-278).  For every row i < num_seqs:
 *   input_ids[i] = sampled[i];  context_lens[i] += 1;
 *   slot_mapping[i] = block_tables[i, (len-1)/block_size] * block_size + (len-1) % block_size  (len = new length)
 *   history[i] = sampled[i] when history != NULL (the host reads all steps' tokens at the end).
 * block_tables int32 [num_seqs, bt_stride] must already list the block the new token falls into; a table
 * that does not sets the slot to -1 and reports B200_ERR_BOUNDS in *status.
 * ------------------------------------------------------------------------------------------- */
int b200_decode_advance(const int64_t* sampled, int64_t* input_ids, int64_t* context_lens,
                        int64_t* slot_mapping, const int32_t* block_tables, int64_t bt_stride,
                        int32_t block_size, int64_t num_blocks, int32_t num_seqs, int64_t* history,
                        int32_t* status, void* stream);

/* Device-resident block tables: writes `count` (row, column, block id) int32 triples into
 * block_tables [rows, bt_stride], so that a decode step uploads only the table entries that changed since
 * the previous step (the reference rebuilds and ships the whole table, engine/model_runner.py:263-268).
 * A triple outside the table is skipped and reported as B200_ERR_BOUNDS in *status. */
int b200_block_table_patch(const int32_t* patches, int32_t count, int32_t* block_tables, int64_t bt_stride,
                           int32_t rows, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Token sampling (Sampler.forward, utils/sampler.py:35-52; greedy argmax of generate.py:62), one launch.
 *   logits [num_rows, >= vocab_size] (row stride in elements) in `dtype`; temperatures fp32 [num_rows] or
 *   NULL (= all greedy).  Row r with temperature T > 0: a draw from softmax(logits[r] / T) as the
 *   exponential race argmax_i (logits_i / T - log E_i), E_i ~ Exp(1) clamped at 1e-10 like the reference;
 *   T <= 0: argmax of the logits, lowest index among equal maxima.  out_tokens int64 [num_rows].
 *   The uniforms are a counter-based function of (seed, offset, row, element): pass a fresh `offset` per
 *   step.  The stream differs from torch's, so only the distribution matches the reference.
 * ------------------------------------------------------------------------------------------- */
int b200_sample(const void* logits, int64_t row_stride, const float* temperatures, int64_t num_rows,
                int32_t vocab_size, uint64_t seed, uint64_t offset, int64_t* out_tokens, int32_t dtype,
                void* stream);

/* ---------------------------------------------------------------------------------------------
 * Greedy head in two launches: the lm_head projection (TransformerLM.lm_head, model/transformer.py:160,183)
 * fused with the greedy argmax of generate.py:62 / the T = 0 rows of the sampler:
 *   tokens[r] = argmax_v bf16( hidden[r] . W[v] + bias[v] ), lowest v among equal maxima,
 * i.e. what argmax over the bf16 logits of a biased linear layer returns, without writing the logits.
 *   hidden [num_rows, k_dim] bf16 contiguous, w [vocab_size, k_dim] bf16, bias [vocab_size] bf16 or NULL,
 *   tokens int64 [num_rows]; workspace of b200_lm_head_argmax_workspace_bytes() bytes, 256-byte aligned
 *   (per-tile maxima; nothing survives the call).  tcgen05 kernel that streams W once; bf16 only, k_dim % 8 == 0.
 * ------------------------------------------------------------------------------------------- */
size_t b200_lm_head_argmax_workspace_bytes(int32_t num_rows, int32_t vocab_size);
int b200_lm_head_argmax(const void* hidden, const void* w, const void* bias, int64_t* tokens, int32_t num_rows,
                        int32_t vocab_size, int32_t k_dim, void* workspace, size_t workspace_bytes,
                        int32_t dtype, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Diagnostic (no counterpart in the reference, which has no device code): runs the give-up path of the
 * bounded barrier waits that the tcgen05 / TMA kernels share.  One CTA holds tensor memory, arms a barrier
 * that can never complete, and waits on it from two threads: one with `poll_limit` polls (1..65536), one
 * with the kernels' default limit.  Nothing faults and nothing loops without bound.  Afterwards
 *   result[0] = 0 and result[1] = poll_limit : the short wait ran out at its limit,
 *   result[2] = 0 and result[3] < 2^22       : the other wait left through the CTA's abort flag,
 *   result[4] = 1                            : tensor memory was allocated and has been freed,
 * and *status holds B200_ERR_TIMEOUT (read and clear it with b200_read_status).  result: device int32[5].
 * ------------------------------------------------------------------------------------------- */
int b200_selftest_bounded_wait(int32_t poll_limit, int32_t* result, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200LLM_H_ */
