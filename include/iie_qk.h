/* C-ABI of libnmc_qk_cuda.so: the B200 (sm_100a) producer of the integer MoE block and the fused
 * Q4_K/Q6_K-dequant integer matmul.
 *
 * Part 1 declares the entry points the reference's ctypes bridge binds (north-mini-code/src/nmc/
 * qk_cuda.py:39-72 lists the required names, :110-214 their argument types); each declaration cites
 * the reference definition it replaces (file:line in north-mini-code/tools/nmc_qk_cuda.cu).  All
 * pointers in part 1 are HOST pointers owned by the caller for the duration of the call; results
 * are byte-identical to the reference CPU oracle.  Return codes: 0 ok, 1 bad argument / runtime
 * failure, 2 wrong quantisation type for a type-specific entry, 3 input outside the exact envelope
 * (caller falls back to its host path).
 *
 * Part 2 declares additive device-pointer entry points (no counterpart in the reference) so that a
 * caller holding tensors in device memory (e.g. PyTorch) never bounces through the host.
 *
 * qtype: 0 = Q4_K (144-byte blocks), 1 = Q6_K (210-byte blocks), 2 = dense int64 (register_i64).
 */
#ifndef IIE_QK_H
#define IIE_QK_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------
 * Part 1: reference ABI v5
 * ---------------------------------------------------------------------------------------------- */
int qk_cuda_abi_version(void);                       /* nmc_qk_cuda.cu:755  returns 5 */
int qk_cuda_available(void);                         /* nmc_qk_cuda.cu:2348 0 = a usable GPU is present */

/* out[t,o] = floor(sum_i W[o,i]*x[t,i] / 2^fw) from raw blocks.               nmc_qk_cuda.cu:720 */
int qk_linear_cuda(const uint8_t *W, const int64_t *x, long long T, long long out_f, long long n_blocks,
                   int fw, int qtype, int64_t *out);

/* Resident weights: handle >= 0, or -1.                                        nmc_qk_cuda.cu:1040-1108 */
int qk_resident_reserve(long long count);
long long qk_register_weight(const uint8_t *W, long long out_f, long long n_blocks, int qtype);
long long qk_register_i64(const int64_t *W, long long rows, long long cols);
long long qk_resident_count(void);                   /* nmc_qk_cuda.cu:1805 */
long long qk_resident_capacity(void);                /* nmc_qk_cuda.cu:1806 */
void qk_free_all(void);                              /* nmc_qk_cuda.cu:1783 */

/* nmc_qk_cuda.cu:1252 */
int qk_apply_resident(long long h, const int64_t *x, long long T, int fw, int64_t *out);
/* Same input through up to 16 weights, outputs concatenated in handle order.   nmc_qk_cuda.cu:1284 */
int qk_apply_resident_grouped(const long long *handles, const int *phase_ids, int count, const int64_t *x,
                              long long T, int fw, long long output_capacity, int64_t *out);
/* Type-specific applies (rc 2 on the other type); Ln is accepted and ignored: the eight-limb
 * decomposition used here is exact for every magnitude the limb rule admits.   nmc_qk_cuda.cu:1932,2003 */
int qk_apply_resident_q6k_dp4a(long long h, const int64_t *x, long long T, int fw, int Ln, int64_t *out);
int qk_apply_resident_q4k_dp4a(long long h, const int64_t *x, long long T, int fw, int Ln, int64_t *out);

/* RMSNorm -> dense int64 router -> top-k (low index on ties) -> sigmoid gates.  nmc_qk_cuda.cu:1116 */
int qk_rmsnorm_router(long long gain_h, long long router_h, const int64_t *x, long long rows, int fa, int fw,
                      unsigned long long eps, int used, long long h_capacity, long long route_capacity,
                      int64_t *h_out, int *ids_out, int64_t *gates_out);

/* Decode MoE FFN on one token over n_e selected experts.                       nmc_qk_cuda.cu:1816,2110 */
int qk_moe_ffn(const long long *gate_h, const long long *up_h, const long long *down_h, int n_e, const int64_t *h,
               const int64_t *gates, long long d_model, long long e_ffn, int fa, int fw, int64_t *out);
int qk_moe_ffn_dp4a(const long long *gate_h, const long long *up_h, const long long *down_h, int n_e,
                    const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa, int fw,
                    int64_t *out);
/* Batched MoE FFN over m*k (token, expert) pairs, token-major handles.         nmc_qk_cuda.cu:2203,2261 */
int qk_moe_ffn_batched(const long long *gate_h, const long long *up_h, const long long *down_h, int m, int k,
                       const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa, int fw,
                       int64_t *out);
int qk_moe_ffn_batched_dp4a(const long long *gate_h, const long long *up_h, const long long *down_h, int m, int k,
                            const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa,
                            int fw, int64_t *out);

long long qk_moe_workspace_allocations(void);        /* nmc_qk_cuda.cu:1807 */
unsigned long long qk_moe_workspace_bytes(void);     /* nmc_qk_cuda.cu:1808 */
void qk_moe_workspace_release(void);                 /* nmc_qk_cuda.cu:1223 */

void qk_profile_reset(void);                         /* nmc_qk_cuda.cu:82 */
void qk_profile_set_enabled(int enabled);            /* nmc_qk_cuda.cu:85 */
int qk_profile_snapshot(unsigned long long *out, int capacity);   /* nmc_qk_cuda.cu:86, 28 counters */

/* Request-scoped attention bank: per-layer K/V rows on the device and the single-token attention sublayer
 * (Q/K/V products of a normalised hidden row, optional interleaved RoPE at position = rows held, K/V append, exact
 * integer softmax attention over the rows held, O product).      nmc_qk_cuda.cu:877,914,927,1363,1530,1765
 *   create  -> handle >= 0, or -1 (bad dimensions, an attention shape the kernels do not cover, out of memory)
 *   import  -> host K/V [n_kv][length][head_dim] int64 of a prefill; rows are held as int32: after a value outside
 *              int32 the next apply on that layer reports the guard (rc 3), where the reference holds int64 and
 *              guards the products
 *   apply   -> x [d_model] and out [>= d_model] are host rows; window -1 = attend to everything, > 0 = that many most
 *              recent rows; rc 0 ok (the layer then holds one more row), 1 bad argument or CUDA failure, 3 an exact
 *              envelope guard fired (K/V beyond int32 or an activation beyond eight base-256 digits); after 1 or 3 from
 *              queued work the layer is poisoned until qk_attention_bank_reset
 * The retained-layer executor entries (moe_configure, moe_bind, moe_begin, moe_continue, moe_export;
 * nmc_qk_cuda.cu:935,984,1557,1658,1748) serve the case where the experts do not all fit on the device; they exist so
 * that the reference bridge accepts the library and report failure (rc 1). */
long long qk_attention_bank_create(int n_layers, long long max_length, long long d_model, int heads, int n_kv,
                                   int head_dim, int fa, const int64_t *cos, const int64_t *sin);
int qk_attention_bank_reset(long long h);
void qk_attention_bank_destroy(long long h);
int qk_attention_bank_moe_configure(long long h, int layer, int experts, int used, long long d_model,
                                    long long expert_ffn);
int qk_attention_bank_moe_bind(long long h, int layer, int expert, long long gate_h, long long up_h,
                               long long down_h);
int qk_attention_bank_import(long long h, int layer, const int64_t *k, const int64_t *v, long long length);
int qk_attention_bank_apply(long long h, int layer, long long qh, long long kh, long long vh, long long oh,
                            const int64_t *x, int fw, int window, int rope, long long inv_sqrt,
                            long long output_capacity, int64_t *out);
int qk_attention_bank_moe_begin(long long h, int layer, long long gain_h, long long router_h, long long qh,
                                long long kh, long long vh, long long oh, const int64_t *x, int use_retained, int fw,
                                unsigned long long eps, int window, int rope, long long inv_sqrt, int cold_capacity,
                                int *cold_count_out, int *cold_ids_out);
int qk_attention_bank_moe_continue(long long h, int layer, int fw, int publish, long long output_capacity,
                                   int64_t *out);
int qk_attention_bank_moe_export(long long h, long long output_capacity, int64_t *out);
unsigned long long qk_attention_bank_workspace_bytes(long long h);

/* ------------------------------------------------------------------------------------------------
 * Part 2: device-pointer extension (additive)
 * ---------------------------------------------------------------------------------------------- */
/* Register a weight whose raw blocks already sit in device memory (copied and re-ordered). */
long long iie_register_weight_dev(const void *raw_dev, long long out_f, long long n_blocks, int qtype);
/* Copy a registered weight back to the host in raw GGUF block order (out_f*n_blocks*{144|210} bytes). */
int iie_weight_export(long long h, void *raw_host);

/* One MoE layer with all experts resident: router handle (Q4_K/Q6_K or dense int64) plus
 * n_experts gate/up/down handles.  Returns a layer handle >= 0, or -1. */
long long iie_moe_layer_create(long long router_h, const long long *gate_h, const long long *up_h,
                               const long long *down_h, int n_experts, int top_k, long long d_model,
                               long long e_ffn);
void iie_moe_layer_destroy(long long layer);

/* Whole MoE block on device tensors, asynchronous on `stream` (a cudaStream_t; NULL = the CUDA default
 * stream): router product, top-k + sigmoid gates, dispatch, gate/up with fused SiLU*up, down with
 * fused gate-weighted combine.  h_dev [T,d_model] int64 -> out_dev [T,d_model] int64 (overwritten,
 * or added to when accumulate != 0), ids_dev [T,top_k] int32, gates_dev [T,top_k] int64 (the last
 * two may be NULL).  Inputs outside the exact envelope raise bits in the flag word. */
int iie_moe_forward_dev(long long layer, const int64_t *h_dev, long long T, int fa, int fw, int accumulate,
                        int64_t *out_dev, int *ids_dev, int64_t *gates_dev, void *stream);

/* The block with its normalisation and residual on device tensors: out = moe(x) when gain_h < 0, else
 * out = x + moe(rmsnorm(x, gain)).  A single token with a quantised router takes three launches
 * (fused routing, gate/up, down); out_dev may alias x_dev. */
int iie_moe_block_dev(long long layer, long long gain_h, const int64_t *x_dev, long long T, int fa, int fw,
                      unsigned long long eps, int64_t *out_dev, int *ids_dev, int64_t *gates_dev, void *stream);

/* The same block on HOST buffers in one call (one upload, one download): out = moe(x) when
 * gain_h < 0, else out = x + moe(rmsnorm(x, gain)) -- the parallel-residual form of the reference's
 * MoE block without its attention term.  ids_out / gates_out may be NULL.  rc 3: an input left the
 * exact envelope and nothing was written. */
int iie_moe_block_host(long long layer, long long gain_h, const int64_t *x, long long T, int fa, int fw,
                       unsigned long long eps, int64_t *out, int *ids_out, int64_t *gates_out);

/* The two halves of the block for expert-parallel callers (the reference has no multi-GPU path; these
 * split what Engine._moe does at north-mini-code/src/nmc/engine.py:375-443 at the point where rows change
 * owner).  iie_route_dev: logits of the replicated router (any registered matrix with one row per expert of
 * the WHOLE model), top-k ids (lowest index wins ties) and sigmoid gates for every row.
 * iie_moe_experts_dev: expert stage of `layer`, whose experts are the ids expert_base .. expert_base +
 * n_experts - 1; every row carries `slots` (id, gate) pairs and pairs with other ids are skipped, so the
 * routing arrays can travel unmodified.  out_dev [T,d_model] receives, per row, the sum over this shard's
 * pairs of floor(down * gate / 2^fa) (overwritten, or added to when accumulate != 0). */
int iie_route_dev(long long router_h, int top_k, const int64_t *h_dev, long long T, int fa, int fw, int *ids_dev,
                  int64_t *gates_dev, void *stream);
int iie_moe_experts_dev(long long layer, const int64_t *h_dev, long long T, const int *ids_dev, const int64_t *gates_dev,
                        int slots, int expert_base, int fa, int fw, int accumulate, int64_t *out_dev, void *stream);

/* Attention of ONE new token over an int32 KV cache, on device tensors (the arithmetic of
 * north-mini-code/src/nmc/cohere2.py:324-354 attention_cached with m = 1; in the reference's CUDA library this
 * lives behind qk_attention_bank_apply, north-mini-code/tools/nmc_qk_cuda.cu:1436-1551):
 *   q_dev [n_heads*head_dim], k_dev / v_dev [n_kv*head_dim]  projected rows of the token, before rotation (not modified),
 *   kcache_dev / vcache_dev [n_kv][cache_rows][head_dim] int32, row `pos` is written by this call,
 *   pos_dev != NULL: the position is read from that device cell when the kernels run and `pos` is only an upper
 *   bound of it (sizes the grids), so a captured launch sequence can be replayed for successive tokens,
 *   window > 0: only keys pos-window+1 .. pos are visible; otherwise all keys 0 .. pos,
 *   rope 0 none, 1 interleaved pairs, 2 rotate-half pairs; cos_dev / sin_dev [>= pos+1][head_dim/2] int64 at 2^fa,
 *   inv_sqrt = round(2^fa / sqrt(head_dim)) as the caller's model defines it,
 *   out_dev [n_heads*head_dim] = (softmax(scores) v) >> fa.
 * Flag bit 2 is raised when a key or value does not fit the int32 cache. */
int iie_attn_decode_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                        int32_t *vcache_dev, long long pos, const int *pos_dev, long long window, const int64_t *cos_dev,
                        const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim, long long cache_rows,
                        int fa, long long inv_sqrt, int64_t *out_dev, void *stream);
/* Attention of `tokens` consecutive new tokens at positions start .. start + tokens - 1 (a prefill, or a chunk of one):
 * q_dev [tokens][n_heads*head_dim], k_dev / v_dev [tokens][n_kv*head_dim] before rotation; all K/V rows are appended
 * to the int32 caches first, then every token attends to the rows up to its own position (causal; window > 0 keeps the
 * last `window` rows), with the exact integer softmax of the single-token entry.  out_dev [tokens][n_heads*head_dim].
 * The computation of north-mini-code/src/nmc/cohere2.py:324-354 (attention_cached with m > 1) and of
 * bonsai/src/trinote/infer_int/reference_bonsai.py:656-720 (rope 2, no window).  0 ok, 1 bad argument or CUDA failure;
 * a K/V value outside int32 raises bit 2 of the flag word. */
int iie_attn_prefill_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                         int32_t *vcache_dev, long long start, long long tokens, long long window, const int64_t *cos_dev,
                         const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim, long long cache_rows, int fa,
                         long long inv_sqrt, int64_t *out_dev, void *stream);
/* One whole parallel decoder block for one token: x_dev += attention(h) Wo^T + moe(h), h = rmsnorm(x_dev, gain) (gain_h < 0:
 * h = x_dev), i.e. north-mini-code/src/nmc/cohere2.py:357-383 (block_cached) with Engine._moe (engine.py:375-443) for the
 * expert half.  `layer` is an iie_moe_layer_create handle with a quantised router, wqkv_h the stacked [Wq|Wk|Wv] matrix, the
 * remaining arguments as for iie_attn_block_dev.  Five launches (norm + QKV + router rows, attention, O, gate/up, down; a
 * spare CTA of the O launch ranks the router logits for the last two) against the six of iie_moe_block_dev + iie_attn_block_dev, same bytes.
 * ids_dev / gates_dev (nullable): the selected experts and their gates.  0 ok, 1 bad argument or CUDA failure, 3 a block
 * scale outside the exact envelope, 5 no fused form for this shape (use the two entries). */
int iie_block_dev(long long layer, long long gain_h, long long wqkv_h, long long wo_h, int64_t *x_dev, int32_t *kcache_dev,
                  int32_t *vcache_dev, long long pos, const int *pos_dev, long long window, const int64_t *cos_dev,
                  const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim, long long cache_rows, int fa, int fw,
                  unsigned long long eps, long long inv_sqrt, int *ids_dev, int64_t *gates_dev, void *stream);
/* Batched decode attention: the new tokens of n_seqs independent sequences in one call, every sequence with its own int32
 * caches (sequence i at kcache_dev / vcache_dev + i * seq_stride elements, each [n_kv][cache_rows][head_dim]) and all at the
 * same position pos (sequences decoded in lockstep).  q_dev [n_seqs][n_heads*head_dim], k_dev / v_dev [n_seqs][n_kv*head_dim]
 * before rotation; row pos of every sequence's caches is written; out_dev [n_seqs][n_heads*head_dim].  Arithmetic of the
 * single-token entry per sequence (north-mini-code/src/nmc/cohere2.py:324-354, m = 1); the reference's batched analogue for
 * its 1-bit decoder is attention_decode_batched_kernel (bonsai/tools/bonsai_q1_gpu.cu:1409).  0 ok, 1 bad argument or CUDA
 * failure; a K/V value outside int32 raises bit 2 of the flag word. */
int iie_attn_decode_batch_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                              int32_t *vcache_dev, long long pos, long long n_seqs, long long seq_stride, long long window,
                              const int64_t *cos_dev, const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim,
                              long long cache_rows, int fa, long long inv_sqrt, int64_t *out_dev, void *stream);
/* The attention half of a decoder block for ONE token, accumulated into the residual row:
 *   x_dev [d_model] += (attention(q, cache) Wo^T), with [q | k | v] = h Wqkv^T,
 * where h is the normalised row whose digit planes the LAST single-token iie_moe_block_dev / iie_moe_forward_dev
 * call left in the library (the reference's block uses the same h for attention and experts, cohere2.py:357-376), so
 * the MoE half of the block must run first.  wqkv_h: one registered matrix with the rows of Wq, Wk, Wv stacked
 * (n_heads*head_dim + 2*n_kv*head_dim rows); wo_h: [d_model, n_heads*head_dim].  Five launches: fused QKV product,
 * the three attention passes, O product.  rc 3: a weight outside the exact envelope.  Other arguments as above. */
int iie_attn_block_dev(long long wqkv_h, long long wo_h, int64_t *x_dev, int32_t *kcache_dev, int32_t *vcache_dev, long long pos,
                       const int *pos_dev, long long window, const int64_t *cos_dev, const int64_t *sin_dev, int rope,
                       int n_heads, int n_kv, int head_dim, long long cache_rows, int fa, int fw, long long inv_sqrt,
                       void *stream);
/* Form of the single-token attention: 1 (default) one cooperative launch when all of its CTAs fit on the device at
 * once (about 4700 visible keys per KV head on B200), else three launches; 0: always three launches.  Same bytes in
 * either form; the switch exists so that tests reach both. */
void iie_set_attn_fused(int enabled);
/* Prefill attention by sixteen-token tiles: 1 (default) both products on tcgen05, 0 on mma.sync (the form that also takes
 * key spans beyond what the int32 TMEM accumulators of the tcgen05 form carry), -1 no tiles (the per-token kernels). */
void iie_set_attn_tile_tc(int enabled);
/* Whole decode step of the MoE decoder in ONE launch: every block of the model (RMSNorm, fused Q/K/V product, rotation,
 * cache append, exact softmax attention, O product, router, top-k, sigmoid gates, gate/up with integer SiLU, down with
 * gate-weighted combine; x += attention + moe) inside a persistent cooperative kernel, one CTA per SM, weights and cache
 * rows streamed through shared-memory rings that run ahead of the arithmetic across the blocks.  Same bytes as the
 * per-block entries (iie_moe_block_dev + iie_attn_block_dev), i.e. as north-mini-code/src/nmc/cohere2.py:357-376
 * (block_cached, one new token) applied layer after layer (cohere2.py:379-383).
 *   iie_decoder_create: model-wide shape; cos_dev / sin_dev [cache_rows][head_dim/2] int64 at 2^fa stay owned by the caller.
 *   iie_decoder_set_layer: block li = norm gain (dense int64 handle), MoE layer (iie_moe_layer_create, with its router),
 *     stacked Wq|Wk|Wv and Wo handles, int32 caches [n_kv][cache_rows][head_dim], full != 0: the block sees every key and
 *     does not rotate (sliding window + interleaved RoPE otherwise).  rc 5: outside what the one-launch kernel carries
 *     (quantisation types other than Q4_K for router / attention / gate / up, large block scales, d_model > 2048, more than
 *     eight query heads per KV head ...): the caller keeps the per-block entries.
 *   iie_decoder_step_dev: x_dev [d_model] is the residual row, updated in place through all blocks; the position is read from
 *     *pos_dev when the kernel runs (pos_bound is its host upper bound and sizes nothing but the checks), or is pos_bound
 *     when pos_dev is NULL.  ids_out_dev / gates_out_dev (optional, [n_layers][top_k]) receive every block's routing.
 *     rc 5: the visible cache rows at pos_bound exceed what one launch holds (about 4300 per KV head on 148 SMs, head_dim 128).
 *     Flag bits raised on the device: 0 digit envelope, 1 RMSNorm envelope, 2 K/V beyond int32, 3 a bounded wait gave up,
 *     4 position cell beyond pos_bound or the cache, 5 a rotated query value beyond int32.
 * The scratch of a decoder is its own (allocated at the first step, fixed size), so a captured step stays valid whatever the
 * library's shared workspaces do. */
long long iie_decoder_create(int n_layers, int n_heads, int n_kv, int head_dim, long long window, long long cache_rows, int fa,
                             int fw, unsigned long long eps, long long inv_sqrt, const int64_t *cos_dev, const int64_t *sin_dev);
int iie_decoder_set_layer(long long dec, int li, long long gain_h, long long moe_layer, long long wqkv_h, long long wo_h,
                          int32_t *kcache_dev, int32_t *vcache_dev, int full);
int iie_decoder_step_dev(long long dec, int64_t *x_dev, long long pos_bound, const int *pos_dev, int *ids_out_dev,
                         int64_t *gates_out_dev, void *stream);
void iie_decoder_destroy(long long dec);

/* Row `token` (or *token_dev when token_dev != NULL) of a registered Q4_K / Q6_K matrix as int64 at 2^frac:
 * the embedding look-up (north-mini-code/src/nmc/engine.py:239-243). */
int iie_embed_dev(long long h, const int *token_dev, long long token, int frac, int64_t *out_dev, void *stream);
/* Index of the largest of n int64 values, lowest index on ties (greedy pick of engine.py:585). */
int iie_argmax_dev(const int64_t *x_dev, long long n, int *out_dev, void *stream);
/* The same for a batch of sequences in one launch each: rows tokens_dev[i] of the matrix -> out_dev[i][width], and the
 * arg-max of each of `rows` rows of n values -> out_dev[i] (a token id of the embedding outside the matrix is the
 * caller's error: ids come from iie_argmax_rows_dev over the same vocabulary). */
int iie_embed_rows_dev(long long h, const int *tokens_dev, int rows, int frac, int64_t *out_dev, void *stream);
int iie_argmax_rows_dev(const int64_t *x_dev, long long rows, long long n, int *out_dev, void *stream);

/* Plain resident product on device tensors: out_dev [T,out_f] = floor(x_dev W^T / 2^fw). */
int iie_apply_dev(long long h, const int64_t *x_dev, long long T, int fw, int64_t *out_dev, void *stream);

/* Integer RMSNorm on device tensors: out = ((x << fa) // isqrt(sum(x^2)//width + eps)) * gain >> fa.
 * gain_h is a dense int64 handle of one row, or -1 for no gain.  Rows outside the exact envelope
 * raise flag bit 1.  (Arithmetic of north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72.) */
int iie_rmsnorm_dev(long long gain_h, const int64_t *x_dev, long long rows, long long width, int fa,
                    unsigned long long eps, int64_t *out_dev, void *stream);

/* Profiling hooks: restrict iie_moe_forward_dev to a subset of its stages (bit 0 limb planes,
 * 1 router product, 2 top-k, 3 gate/up, 4 down; 0 = all) so that one kernel can be timed alone on
 * data left by a previous full call; and the number of kernels launched since load. */
void iie_profile_stage_mask(int mask);
/* Switch programmatic dependent launch between the three single-token kernels on (default) or off. */
void iie_set_pdl(int enabled);
/* Token count from which iie_moe_forward_dev uses the tcgen05 grouped GEMMs instead of the streamed
 * kernels (default 32; a very large value disables the tensor-core path). */
void iie_set_tc_min_tokens(long long tokens);
unsigned long long iie_launch_count(void);
/* Launches of each tensor-core (tcgen05) tile shape since load, so a test can tell which shape served a call:
 * out[0..6] = Q4_K gate/up with 3 / 4 activation digits, Q6_K down with 5 / 6, Q4_K down with 5, Q4_K linear with
 * 3 / 5.  Returns 7, or -1 when capacity < 7. */
int iie_prefill_launch_counts(unsigned long long *out, int capacity);
/* Workspace generation: changes whenever a scratch buffer of the library is freed (to grow, by
 * qk_moe_workspace_release or qk_free_all).  A CUDA graph captured over iie_*_dev calls holds the scratch addresses of
 * its capture; record this value at capture and refuse to replay once it has changed. */
unsigned long long iie_workspace_generation(void);

/* iie_apply_dev without any allocation (no counterpart in the reference).  For callers that cannot let
 * a library allocate device memory at call time: a process whose own pool already holds the whole
 * device, or a latency-critical loop that cannot take the implicit synchronisation of cudaMalloc.
 * The limb planes of the activation live in a 4 MiB array inside the library image (held by every GPU
 * that loads the library until exit), so T * 8 * in_features must not exceed 4 194 304 bytes
 * (e.g. T <= 256 at 2048 input features); larger requests return 4 and do nothing.  The first call
 * on a device looks up the array's device address; make that call before starting any stream
 * capture.  All calls share the array: two calls that overlap on the GPU race.  Same results and
 * flag bits as iie_apply_dev. */
int iie_apply_dev_static(long long h, const int64_t *x_dev, long long T, int fw, int64_t *out_dev, void *stream);

/* Read and clear the device flag word (synchronises the library stream and `stream`):
 * bit 0 an activation left the 8-limb envelope, bit 1 RMSNorm envelope, bit 2 dense router sum. */
int iie_flags_read_clear(void *stream);

#ifdef __cplusplus
}
#endif
#endif
