/* C-ABI of the Q1_0 (1-bit weights) dense path.
 *
 * Part 1 re-exports, with identical names, argument order and return codes, the entry points that the
 * reference bridge bonsai/src/trinote/infer_int/gpu_native.py:44-185 binds from libbonsai_q1_gpu.so
 * (implemented there in bonsai/tools/bonsai_q1_gpu.cu).  All pointers in part 1 are HOST pointers and
 * every call synchronises before it returns.  Arrays are C-contiguous:
 *     x      [tokens][n_blocks*128]  int64     activations at scale 2^frac
 *     bits   [out_f][n_blocks][16]   uint8     sign bits, little-endian inside a byte, 1 -> +1, 0 -> -1
 *     scale  [out_f][n_blocks]       int64 (or int32 for the *_i32 registrations)
 *     out    [tokens][out_f]         int64
 *     out[t,o] = sum_b floor( ((sum_i +-x[t,128b+i]) * scale[o,b] mod 2^64) / 2^frac )   (mod 2^64)
 * Return codes: 0 ok, 1 bad arguments, 2 CUDA failure, 4 outside the caller-chosen digit envelope.
 *
 * Part 2 is additive (device pointers, no reference counterpart).
 */
#ifndef IIE_Q1_H
#define IIE_Q1_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- part 1: the reference's names ---------------------------------------------------------------- */

/* bonsai_q1_gpu.cu:1970 - ABI generation the bridge may probe (3). */
int bonsai_gpu_abi_version(void);
/* bonsai_q1_gpu.cu:1974,1978 - code and text of the calling thread's last failure ("ok" when none). */
int bonsai_gpu_last_error_code(void);
const char *bonsai_gpu_last_error(void);
/* bonsai_q1_gpu.cu:2032 - 0 iff a usable CUDA device exists. */
int bonsai_gpu_available(void);
/* bonsai_q1_gpu.cu:2041 - free / total device memory as the allocator sees it; 0 ok, 1 null, 2 CUDA. */
int bonsai_gpu_mem_info(unsigned long long *free_bytes, unsigned long long *total_bytes);
/* bonsai_q1_gpu.cu:2073 - bytes of bits + scales registered so far (as handed in, before re-ordering). */
unsigned long long bonsai_q1_resident_weight_bytes(void);

/* bonsai_q1_gpu.cu:2200 - one-shot product: uploads the weight, multiplies, downloads. */
int bonsai_q1_linear_gpu(const long long *x, const unsigned char *bits, const long long *scale, long long tokens,
                         long long out_f, long long n_blocks, long long frac, long long *out);
/* bonsai_q1_gpu.cu:2245 - same product through the digit path; |L| in 1..8 is the number of base-256
 * digits the caller vouches for (a negative L only selected another kernel shape in the reference).
 * Every L computes with all eight digits here; rc 4 when an activation needs more than |L| < 8 digits,
 * as the reference's L = 4 range guard reports. */
int bonsai_q1_linear_dp4a_gpu(const long long *x, const unsigned char *bits, const long long *scale, long long tokens,
                              long long out_f, long long n_blocks, long long frac, int L, long long *out);

/* bonsai_q1_gpu.cu:2308,2329,2350,2368 - upload once, returns a handle >= 0 or -1.  The three int32
 * variants differ only in the device layout the reference chose; here every registration is stored
 * in the same tensor-core order. */
long long bonsai_q1_register_weight(const unsigned char *bits, const long long *scale, long long out_f, long long n_blocks);
long long bonsai_q1_register_weight_i32(const unsigned char *bits, const int *scale, long long out_f, long long n_blocks);
long long bonsai_q1_register_weight_i32_gpu_layout(const unsigned char *bits, const int *scale, long long out_f,
                                                   long long n_blocks);
long long bonsai_q1_register_weight_i32_bmma(const unsigned char *bits, const int *scale, long long out_f,
                                             long long n_blocks);
/* bonsai_q1_gpu.cu:2388 - product with a registered weight. */
int bonsai_q1_apply_resident(long long handle, const long long *x, long long tokens, long long frac, long long *out);
/* bonsai_q1_gpu.cu:3659 - drop every registered weight; handles start again at 0. */
void bonsai_q1_free_weights(void);

/* bonsai_q1_gpu.cu:2428 - RMSNorm of fixed-point rows, gain nullable.  0 ok, 1 bad arguments or CUDA
 * failure, 4 a row left the exact envelope (the caller recomputes on its big-integer path). */
int bonsai_rmsnorm_gpu(const long long *x, long long rows, long long cols, long long frac, long long eps,
                       const long long *gain, long long *out);

/* ---- part 1b: whole-model entries (the bridge treats each as optional, gpu_native.py:53-170) ------------------
 * Layouts are the reference's: q [H][M][hd], K/V [Hkv][L][hd], caches of the decode context [n_layers][Hkv][Lb][hd]
 * per sequence, all int64 host arrays.  On the device K/V rows are int32: a value that does not fit gives the
 * overflow status on which the bridge redoes the call on the host (2 for the two attention entries, 4 for the model
 * entries), like any RMSNorm envelope miss. */

/* bonsai_q1_gpu.cu:2020 - upload an int64 array once (gains, rope tables); handle >= 0 or -1.  Released by
 * bonsai_q1_free_weights. */
long long bonsai_buf_upload_i64(const long long *host, long long n);
/* bonsai_q1_gpu.cu:2475 - causal attention of M new tokens at positions start .. start+M-1 over L = start+M keys;
 * q after per-head norm and rotation, k/v the full rows.  out [H][M][hd].  0 ok, 1 bad arguments / CUDA, 2 overflow. */
int bonsai_attention_prefill_gpu(const long long *q, const long long *k, const long long *v, long long H, long long Hkv,
                                 long long hd, long long M, long long L, long long start, long long frac,
                                 long long inv_sqrt_fp, long long *out);
/* bonsai_q1_gpu.cu:2550 - one new token of each of B sequences: q [B][H][hd], caches [B][Hkv][cap][hd] padded,
 * lengths [B] = valid rows of each sequence (the new token's row included).  out [B][H][hd].  0 / 1 / 2 as above. */
int bonsai_attention_decode_batched_gpu(const long long *q, const long long *Kc, const long long *Vc, const long long *lengths,
                                        long long B, long long H, long long Hkv, long long hd, long long cap, long long frac,
                                        long long inv_sqrt_fp, long long *out);
/* bonsai_q1_gpu.cu:3694 - the whole prefill on the device: x_embed [T][d] -> every layer -> final norm and output matrix
 * on the last row -> out_logits [vocab].  wq .. w2: per-layer weight handles; n1g .. kng: per-layer buffer handles of the
 * gains; finalg, cos_h, sin_h buffer handles; out_head a weight handle.  out_k / out_v (nullable): the K (after head
 * norm and rotation) and V rows of every layer, [n_layers][Hkv][T][hd].  0 ok, 1 bad arguments / CUDA, 4 overflow. */
int bonsai_prefill_forward_gpu(const long long *x_embed, long long T, long long d, long long n_layers, long long H, long long Hkv,
                               long long hd, long long dff, long long frac, long long eps, long long inv_sqrt_fp,
                               const long long *wq, const long long *wk, const long long *wv, const long long *wo,
                               const long long *w1, const long long *wu, const long long *w2, const long long *n1g,
                               const long long *n2g, const long long *qng, const long long *kng, long long finalg,
                               long long out_head, long long cos_h, long long sin_h, long long *out_logits, long long *out_k,
                               long long *out_v);
/* bonsai_q1_gpu.cu:3517,3565,3588,3649 - decode context of B sequences with device K/V of `cap` rows each: create
 * (handle >= 0 or -1), seed sequence b with the K/V rows of its prefill, one decode step for all sequences
 * (x_in [B][d] the new tokens' embedded rows, pos [B] each sequence's position = rows cached before the step,
 * out_logits [B][vocab]; 0 ok, 1 bad arguments / CUDA, 4 overflow), free. */
long long bonsai_decode_ctx_create(long long B, long long n_layers, long long H, long long Hkv, long long hd, long long d,
                                   long long dff, long long cap, long long vocab, long long frac, long long eps,
                                   long long inv_sqrt, const long long *wq, const long long *wk, const long long *wv,
                                   const long long *wo, const long long *w1, const long long *wu, const long long *w2,
                                   const long long *n1g, const long long *n2g, const long long *qng, const long long *kng,
                                   long long finalg, long long out_head, long long cos_h, long long sin_h);
int bonsai_decode_ctx_seed_seq(long long ctx_h, long long b, const long long *k_src, const long long *v_src, long long Lb);
int bonsai_decode_step(long long ctx_h, const long long *x_in, const long long *pos, long long *out_logits);
void bonsai_decode_ctx_free(long long ctx_h);

/* ---- part 2: additive, device pointers (no counterpart in the reference) --------------------------- */

/* Product with a registered weight on device buffers, asynchronous on `stream` (NULL = the CUDA default
 * stream).  Scratch for the digit planes is process-global and grows on demand: one caller at a time. */
int iie_q1_apply_dev(long long handle, const int64_t *x_dev, long long tokens, long long frac, int64_t *out_dev,
                     void *stream);
/* Product with the activation step before it and the residual after it in the same two launches:
 *   mode 0: a = x;   mode 1: a = rmsnorm(x, gain_dev, eps 1) (gain_dev NULL = no gain; an envelope violation sets
 *   bit 1 of the flag word iie_flags_read_clear reports);   mode 2: a = ((x * sigmoid(x)) >> frac) * x2 >> frac with
 *   wrapping products, x and x2 rows `ld` apart (reference_bonsai.py:603-615 _ffn_ref).
 *   out = a W^T (+ add_dev when not NULL; add_dev may be out_dev).  x is [tokens][n_blocks*128] (mode 2: row stride ld).
 * 0 ok, 1 bad argument, 2 CUDA failure. */
int iie_q1_apply_fused_dev(long long handle, int mode, const int64_t *x_dev, const int64_t *x2_dev, long long ld,
                           const int64_t *gain_dev, long long tokens, long long frac, const int64_t *add_dev,
                           int64_t *out_dev, void *stream);
/* RMSNorm (eps 1) of rows_a + rows_b consecutive rows of `width` values in one launch: the first rows_a rows with
 * gain_a_dev, the rest with gain_b_dev (the per-head query and key norms of reference_bonsai.py:286-297,672-673).
 * Envelope violations set bit 1 of the flag word.  0 ok, 1 bad argument, 2 CUDA failure. */
int iie_q1_head_norm_dev(const int64_t *x_dev, long long rows_a, long long rows_b, long long width, const int64_t *gain_a_dev,
                         const int64_t *gain_b_dev, long long frac, int64_t *out_dev, void *stream);
/* out = ((gate * sigmoid(gate)) >> frac) * up >> frac, both products modulo 2^64: the SwiGLU of
 * bonsai/src/trinote/infer_int/reference_bonsai.py:246-262 and 611-614.  0 ok, 1 bad argument, 2 CUDA failure. */
int iie_q1_silu_mul_dev(const int64_t *gate_dev, const int64_t *up_dev, long long n, long long frac, int64_t *out_dev,
                        void *stream);
/* One row of a registered weight as int64 (sign * block scale, reference_bonsai.py:138-146 q1_rows_fp): the row index
 * is read from the device cell `row_dev` when that is not NULL, else `row`. */
int iie_q1_embed_dev(long long handle, const int *row_dev, long long row, int64_t *out_dev, void *stream);
/* Launch form of the single-token product: 1 = the run of tiles of a CTA is requested with bulk copies into shared
 * memory up front, 0 (default) = per-lane loads with one tile of look-ahead.  Same results, same speed within 3 %. */
void iie_q1_set_stream(int on);
/* Changes whenever a scratch buffer of the Q1_0 entries is freed (to grow, or by bonsai_q1_free_weights): a CUDA graph
 * captured over iie_q1_*_dev calls holds the old addresses and must be captured again. */
unsigned long long iie_q1_workspace_generation(void);
/* Shape of a registered weight; 0 ok, 1 unknown handle. */
int iie_q1_weight_shape(long long handle, long long *out_f, long long *n_blocks, int *scale_bits);

#ifdef __cplusplus
}
#endif
#endif
