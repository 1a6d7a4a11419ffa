// Host-callable launchers of the CUDA kernels (internal interface between the .cu files).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace iie {

// Number of kernels this library has launched since it was loaded (benchmarks report it).
extern unsigned long long g_launches;
inline void note_launch(unsigned long long n = 1) { __atomic_fetch_add(&g_launches, n, __ATOMIC_RELAXED); }

enum SkinnyMode { MODE_LINEAR = 0, MODE_GATEUP = 1, MODE_DOWN = 2, MODE_FRONT = 3 };

// Arguments of the streamed ("skinny") fused-dequant product.  Work is organised in groups: group g
// uses weight matrix `expert = grp_expert ? grp_expert[g] : g` and owns the activation rows
// ("pairs") [grp_off[g], grp_off[g+1]) (grp_off == nullptr: every group owns exactly pair g... see
// `pairs_per_group`).
struct SkinnyArgs {
    const uint8_t *const *wa;      // per expert: repacked weight (stream A: linear/down weight, or gate)
    const uint8_t *const *wb;      // per expert: stream B (up weight) for MODE_GATEUP, else unused
    const int *grp_expert;         // [n_groups] or nullptr (identity)
    const int *grp_off;            // [n_groups+1] or nullptr (group g owns pairs [g*ppg, (g+1)*ppg))
    int pairs_per_group;           // used when grp_off == nullptr
    long long out_f;               // output rows of the weight matrix
    long long n_blocks;            // 256-column super-blocks per row
    int fw, fa;
    const int8_t *xl;              // activation limb planes [x_row][8][K]
    const int *xidx;               // pair -> x_row, or nullptr (identity)
    int64_t *out;                  // LINEAR: [pair][out_f]; GATEUP: gu [pair][out_f]; DOWN: [token][out_f] accumulated
    int8_t *out_limbs;             // GATEUP: limb planes of gu [pair][8][out_f] (nullable)
    const int64_t *gates;          // DOWN: per-pair gate weight
    const int *pair_tok;           // DOWN: pair -> token row of `out`, or nullptr (token 0)
    int *flags;                    // bit 0: a value left the 8-limb envelope
};

cudaError_t launch_skinny(int qtype, int mode, const SkinnyArgs &a, int n_groups, int max_pairs_per_group,
                          cudaStream_t s);

// Single-token streaming product (stream.cu).  Work = n_sel selected matrices x their 16-row tiles.
struct StreamArgs {
    const uint8_t *const *wa;      // per matrix: repacked weight (linear/down weight, or gate)
    const uint8_t *const *wb;      // per matrix: up weight (MODE_GATEUP)
    const int *sel;                // [n_sel] matrix indices on the device, or nullptr (identity)
    const uint8_t *const *sel_wa;  // optional: [n_sel] already-resolved pointers (then wa/wb/sel are not read)
    const uint8_t *const *sel_wb;
    int n_sel;
    int pdl;                       // 1: launched with programmatic stream serialization (see stream.cu)
    int early_weights;             // 1: the selected-pointer arrays are final before the previous kernel ends
    int tiles_per_expert, tiles_per_cta;   // filled in by the launcher
    long long out_f, n_blocks;
    int fw, fa;
    int fast;                      // fw >= 24 and every block scale below 2^31: 32-bit scale arithmetic
    long long sig_log2e, sig_clip; // sigmoid constants for fa (filled in by the launcher)
    const int8_t *xl;              // limb planes [8][K] (shared) or [n_sel][8][K]
    int x_per_sel;
    const int *x_nl;               // device: limbs in use by x (<= 4 enables the half-column path), or nullptr
    int x_nl_n;                    // how many consecutive cells x_nl points at (their maximum counts; 0 or 1: one cell)
    int64_t *out;                  // LINEAR [n_sel][out_f]; GATEUP gu [n_sel][out_f] (nullable); DOWN [out_f] accumulated
    int8_t *out_limbs;             // GATEUP: limb planes of gu [n_sel][8][out_f]
    int *out_nl;                   // GATEUP: atomicMax of the limbs gu needs
    const int64_t *gates;          // DOWN: [n_sel]
    int *flags;                    // bit 0 limb envelope, bit 3 a copy never arrived
    // Top-k prologue (GATEUP / DOWN, logits != nullptr): every CTA ranks the n_experts router logits itself (lowest index
    // first among equals) and the k best select the matrices of wa / wb; their sigmoid gates weight the DOWN epilogue.
    // `sel`, `sel_wa` and `gates` are then not read.  CTA 0 also stores ids / gates where the pointers are given.
    const int64_t *logits;
    int n_experts;
    int *ids_out;
    int64_t *gates_out;
    // MODE_FRONT: the front of a decoder block in one launch.  Every CTA normalises the row x (RMSNorm with `gain`,
    // digit planes in shared memory), then the CTAs share the rows of two matrices with that one activation:
    // wa[0] (out_f rows -> out) and wb[0] (out_f_b rows -> out_b), e.g. the stacked Q/K/V matrix and the router.
    // CTA 0 also leaves the planes and their digit count for the kernels that follow, and zeroes *gu_nl_zero.
    const int64_t *x, *gain;
    unsigned long long eps;
    long long out_f_b;
    int64_t *out_b;
    int8_t *hl_out;
    int *h_nl_out, *gu_nl_zero;
    // optional: rows [lo, pos) of `pf_heads` row-major tables (the key cache of the attention kernel that follows) are
    // prefetched into L2 while this kernel runs; lo from the window, pos = *pf_pos_dev (or pf_pos), refused beyond pf_pos
    const void *pf_base;
    long long pf_rows, pf_pos, pf_window;
    int pf_heads, pf_row_bytes;
    const int *pf_pos_dev;
    // optional, MODE_DOWN: one CTA beyond those that own tiles ranks rank_n router logits (largest first, lowest index among
    // equals), and leaves the rank_k selected indices and their sigmoid gates in rank_ids / rank_gates (and ids_out / gates_out)
    // for the kernels behind this one.  The logits must be final before the kernel in front of this one started.
    const int64_t *rank_logits;
    int rank_n, rank_k;
    int *rank_ids;
    int64_t *rank_gates;
    // optional: rank_tabs = [3][rank_n] matrix pointers (gate, up, down); the selected ones are left in rank_ptrs [3][rank_k], so
    // that the kernels behind find their weights with one load (their sel_wa / sel_wb)
    const uint8_t *const *rank_tabs;
    const uint8_t **rank_ptrs;
    int tiles_b;                   // filled in by the launcher
};
cudaError_t launch_stream(int qtype, int mode, const StreamArgs &a, cudaStream_t s);

// Fused single-token routing (route.cu): optional RMSNorm, limb planes, quantised router product,
// top-k + sigmoid gates, and initialisation of the block's output row.
struct RouteArgs {
    const int64_t *x;              // [d] input row
    const int64_t *gain;           // [d] RMSNorm gain, or nullptr (no normalisation: h = x)
    int d, fa, fw;
    unsigned long long eps;
    const uint8_t *router;         // repacked quantised router [n_experts, d]
    int router_q, n_experts, k;
    int8_t *hl;                    // out: limb planes of h [8][d]
    int *h_nl;                     // out: limbs in use by h
    int64_t *h_out;                // out (nullable): h as int64
    int64_t *logits;               // scratch [n_experts]
    int *ids;                      // out [k]
    int64_t *gates;                // out [k]
    int64_t *init_out;             // nullable: row to initialise for the down stage
    int init_mode;                 // 0 leave, 1 zero, 2 copy x (residual)
    const uint8_t *const *tabs;    // optional: [3][n_experts] gate/up/down pointer tables of the layer
    const uint8_t **sel_ptrs;      // optional out: [3][k] pointers of the selected experts
    int pdl;                       // 1: launched with programmatic stream serialization
    int *gu_nl;                    // zeroed here for the following gate/up kernel
    unsigned *counter;             // zero-initialised ticket for last-CTA detection (self-resetting)
    int *flags;                    // bit 0 limb envelope, bit 1 RMSNorm envelope
};
cudaError_t launch_route(const RouteArgs &a, cudaStream_t s);

// Grouped products for small batches (batch.cu): group e = expert e with the rows [grp_off[e], grp_off[e+1]).
struct BatchArgs {
    const uint8_t *const *wa;      // per expert: linear / down weight, or gate
    const uint8_t *const *wb;      // per expert: up weight (MODE_GATEUP)
    const int *grp_off;            // device [n_groups + 1]
    int n_groups;
    long long out_f, n_blocks;
    int fw, fa, fast;
    const int8_t *xl;              // digit planes [x_row][8][K]
    const int *xidx;               // pair -> x_row, or nullptr (identity)
    const int *x_nl;               // device: digits in use by x (<= 4 enables the half-column path), or nullptr
    int64_t *out;                  // LINEAR [pair][out_f]; GATEUP gu [pair][out_f] (nullable); DOWN [token][out_f] accumulated
    int8_t *out_limbs;             // GATEUP: digit planes of gu [pair][8][out_f]
    int *out_nl;                   // GATEUP: atomicMax of the digits gu needs
    const int64_t *gates;          // DOWN: per pair
    const int *pair_tok;           // DOWN: pair -> token row
    int *flags;
    int tiles_per_expert, tiles_per_cta;   // filled in by the launcher
    long long sig_log2e, sig_clip;
};
cudaError_t launch_batch(int qtype, int mode, const BatchArgs &a, cudaStream_t s);

// Prefill-regime grouped products on tcgen05 (prefill.cu).  Pairs are sorted by expert: expert x owns
// pairs [grp_off[x], grp_off[x+1]).
struct PrefillArgs {
    const uint8_t *const *wa;      // per expert: repacked weight (down / linear weight, or gate)
    const uint8_t *const *wb;      // per expert: up weight (MODE_GATEUP)
    const int *grp_off;            // [n_experts + 1]
    int n_experts;
    long long n_pairs;             // total pairs (bounds the grid)
    long long out_f, n_blocks;
    int fw, fa;
    int n_ntiles;                  // filled in by the launcher
    long long sig_log2e, sig_clip;
    const int8_t *xl;              // activation limb planes [x_row][8][K]
    const int *xidx;               // pair -> x_row, or nullptr (identity)
    int8_t *xg;                    // with xidx: scratch for the planes gathered into pair order, n_pairs * 4 * K bytes
    int64_t *out;                  // GATEUP: gu [pair][out_f] (nullable); DOWN: [token][out_f] accumulated; LINEAR [pair][out_f]
    int8_t *out_limbs;             // GATEUP: limb planes of gu [pair][8][out_f]
    int *out_nl;                   // GATEUP: atomicMax of the limbs gu needs
    const int64_t *gates;          // DOWN: per pair
    const int *pair_tok;           // DOWN: pair -> token row
    int *flags;
};
cudaError_t launch_prefill(int qtype, int mode, int nl, const PrefillArgs &a, cudaStream_t s);
// launches of each tensor-core tile shape since the library was loaded, in the order: Q4_K gate/up with 3 / 4 activation
// digits, Q6_K down with 5 / 6, Q4_K down with 5, Q4_K linear with 3 / 5
constexpr int PF_SHAPES = 7;
extern unsigned long long g_prefill_launches[PF_SHAPES];

// Re-order raw GGUF blocks into the half-tile layout; also reduces max |d| and max |dmin| half bit
// patterns (sign stripped) into maxbits[0..1] (device memory, caller zeroes).
cudaError_t launch_repack(const uint8_t *raw, uint8_t *dst, long long out_f, long long n_blocks, int qtype,
                          unsigned *maxbits, cudaStream_t s);
// Inverse of launch_repack (used by tests and by weight export).
cudaError_t launch_unpack(const uint8_t *src, uint8_t *raw, long long out_f, long long n_blocks, int qtype,
                          cudaStream_t s);

// int64 rows -> balanced base-256 limb planes [row][8][K]; sets flags bit 0 on overflow.
cudaError_t launch_limbs(const int64_t *x, long long n_rows, long long K, int8_t *planes, int *flags, cudaStream_t s,
                         int *nl_out = nullptr);   // nl_out: atomicMax of the limbs in use (caller zeroes)

// p[0] = a, p[1] = b on the stream (kernel arguments travel by value, so a captured launch replays correctly where a
// copy from a host stack variable would not)
cudaError_t launch_set2(int *p, int a, int b, cudaStream_t s);

// cold[0] = number of ids whose `bound` byte is 0, cold[1..] = those ids in order; an id outside [0, n_experts) raises flag bit 1
cudaError_t launch_cold_routes(const int *ids, int k, const unsigned char *bound, int n_experts, int *cold, int *flags, cudaStream_t s);
// out = a + b (wrapping), out may alias either input
cudaError_t launch_add_rows(const int64_t *a, const int64_t *b, int64_t *out, long long n, cudaStream_t s);

// Exact 128-bit reference-order product for inputs outside the fast envelope: out[pair][o].
cudaError_t launch_exact_linear(const uint8_t *w, int qtype, long long out_f, long long n_blocks, const int64_t *x,
                                long long T, int fw, int64_t *out, cudaStream_t s);
cudaError_t launch_exact_dense(const int64_t *w, long long out_f, long long in_f, const int64_t *x, long long T,
                               int fw, int64_t *out, int *flags, cudaStream_t s);

// a[i] = (silu(a[i]) * b[i]) >> fa
cudaError_t launch_silu_mul(int64_t *a, const int64_t *b, long long n, int fa, cudaStream_t s);
// out[t][o] (+)= sum_j (dn[(t*k+j)][o] * gates[t*k+j]) >> fa
cudaError_t launch_combine(const int64_t *dn, const int64_t *gates, long long T, int k, long long d_model, int fa,
                           int64_t *out, cudaStream_t s);

// Top-k (descending, lowest index on ties) + sigmoid gates; one warp per row.  n_experts <= 1024.
cudaError_t launch_topk(const int64_t *logits, long long rows, int n_experts, int k, int fa, int *ids,
                        int64_t *gates, cudaStream_t s);

// Integer RMSNorm with optional gain; flags bit 1 set when a row leaves the exact envelope.
cudaError_t launch_rmsnorm(const int64_t *x, long long rows, long long width, const int64_t *gain, int fa,
                           unsigned long long eps, int64_t *out, int *flags, cudaStream_t s);
// the same with the normalised rows also (out may be NULL: only) written as Q1_0 activation operands: digit planes
// [row][8][width] and 128-element block sums [row][width/128]; width must be a multiple of 128
cudaError_t launch_rmsnorm_planes(const int64_t *x, long long rows, long long width, const int64_t *gain, int fa,
                                  unsigned long long eps, int64_t *out, int8_t *planes, int64_t *totals, int *flags, cudaStream_t s);

// Counting-sort dispatch of (token, slot) pairs by expert (single CTA, n_experts <= 1024).
//   ids [T*k], gates [T*k] -> grp_off [E+1], pair_tok [T*k] (token of each sorted pair),
//   pair_gate [T*k] (its gate weight).  Expert e of this shard is id expert_base + e; other ids are dropped.
cudaError_t launch_dispatch(const int *ids, const int64_t *gates, long long T, int k, int n_experts, int *grp_off,
                            int *pair_tok, int64_t *pair_gate, cudaStream_t s, int expert_base = 0);

// One new token's attention over an int32 KV cache (attn.cu): rotation, cache append, three softmax passes.
struct AttnArgs {
    const int64_t *q;              // [H*hd] projected query (rotated on the fly, not modified)
    const int64_t *k, *v;          // [Hkv*hd] projected key / value of the new token
    int32_t *kcache, *vcache;      // [Hkv][Lmax][hd]
    long long pos, lo, Lmax;       // position of the new token (an upper bound when pos_dev is set), first visible key
                                   // (computed on the device), cache rows
    const int *pos_dev;            // optional: the position in device memory (for replayed graphs)
    long long window;              // > 0: only the last `window` keys are visible
    const int64_t *cos, *sin;      // [>= pos+1][hd/2] at 2^fa, or nullptr when rope == 0
    int rope;                      // 0 none, 1 interleaved pairs (2i, 2i+1), 2 rotate-half pairs (i, i + hd/2)
    int H, Hkv, hd, fa;
    long long inv_sqrt, log2e, clip;
    int64_t *scores;               // scratch [H][Lmax]
    int32_t *e;                    // scratch [H][Lmax]
    long long *hmax;               // scratch [H]
    unsigned long long *Z;         // scratch [H]
    long long *acc;                // scratch [H][hd]
    unsigned *ticket;              // scratch
    long long *partial;            // scratch [ceil(Lmax/64)][Hkv][H/Hkv][hd]: per-chunk partial sums of the one-launch form
    int64_t *out;                  // [H*hd], nullable
    int8_t *out_limbs;             // nullable: digit planes [8][H*hd] of the result
    int *out_nl;                   // nullable: digits in use by the result (the one-CTA-per-SM decode form leaves one count per KV head: out_nl[kv])
    int pdl;                       // 1: the one-launch form is launched with programmatic stream serialization
    int *flags;                    // bit 0 digit envelope, bit 2 a key / value does not fit the int32 cache
    int batch;                     // > 0: that many consecutive new tokens (prefill); q, k, v, out then hold one row per token,
                                   // pos is the position of the first, the scratch holds one set of statistics per token
    long long Ls;                  // row stride of scores / e (0: Lmax)
    long long seq_stride;          // with batch > 0: elements between the caches of consecutive sequences (batched decode: token i is
                                   // sequence i's new token, all at position pos); 0: the tokens are consecutive positions of one sequence
    int chunk;                     // keys per CTA of the one-CTA-per-SM form (filled in by the launcher)
    int pv_splits;                 // batch > 0: CTAs that share the key chunks of one (token, KV head) pair (0 / 1: one)
    long long *pv_part;            // scratch [batch][pv_splits][H][hd] for their raw sums
};
cudaError_t launch_attn_decode(const AttnArgs &a, cudaStream_t s);
// `batch` new tokens at positions pos .. pos + batch - 1 against the cache rows before them and each other (causal):
// all K/V rows are appended first, then scores, exponentials and the probability-value sums run per token
cudaError_t launch_attn_prefill(const AttnArgs &a, cudaStream_t s);
extern int g_attn_fused;           // 1: one cooperative launch when it fits, 0: three launches
// passes 1 and 3 of a prefill by tiles of sixteen tokens on the tensor cores (attn_tile.cu), for the shapes attn_tiles_ok accepts
bool attn_tiles_ok(const AttnArgs &a);
extern int g_attn_tile_tc;         // 1: the tile products on tcgen05 (the default), 0: on mma.sync, -1: no tiles
cudaError_t launch_attn_tile_scores(const AttnArgs &a, cudaStream_t s);
cudaError_t launch_attn_tile_exp(const AttnArgs &a, cudaStream_t s);
cudaError_t launch_attn_tile_pv(const AttnArgs &a, cudaStream_t s);
// hmax = INT64_MIN, Z = acc = ticket = 0: once after the statistics buffer is (re)allocated; every call leaves them so
cudaError_t launch_attn_reset(long long *hmax, unsigned long long *Z, long long *acc, unsigned *ticket, int H, int hd, cudaStream_t s);
cudaError_t launch_embed_row(const uint8_t *w, int qtype, long long nb, const int *row_dev, long long row_host, int frac,
                             int64_t *out, cudaStream_t s);
cudaError_t launch_argmax(const int64_t *x, long long n, int *out, cudaStream_t s);
// the same for many rows in one launch: rows_dev[i] -> out[i][nb * 256]; arg-max of each of `rows` rows of n values
cudaError_t launch_embed_rows(const uint8_t *w, int qtype, long long nb, const int *rows_dev, int n_rows, int frac, int64_t *out, cudaStream_t s);
cudaError_t launch_argmax_rows(const int64_t *x, long long rows, long long n, int *out, cudaStream_t s);

// Whole decode step as one persistent cooperative kernel (decode.cu).
struct DecodeLayer {
    const int64_t *gain;           // [d] RMSNorm gain of the block
    const uint8_t *router;         // repacked Q4_K [E, d]
    const uint8_t *wqkv;           // repacked Q4_K [(H + 2 Hkv) * hd, d]: rows of Wq, Wk, Wv stacked
    const uint8_t *wo;             // repacked Q4_K [d, H * hd]
    const uint8_t *const *tabs;    // device [3][E]: gate, up, down pointers of the block's experts
    int32_t *kcache, *vcache;      // [Hkv][Lmax][hd]
    int full;                      // 1: attends to every key, no rotation; 0: sliding window + interleaved RoPE
    int down_q;                    // quantisation type of the down matrices
};
struct DecodeArgs {
    const DecodeLayer *layers;     // device [n_layers]
    int n_layers;
    int d, H, Hkv, hd, E, k, eff, fa, fw;
    unsigned long long eps;
    long long window, Lmax;
    const int64_t *cos, *sin;      // [Lmax][hd/2] at 2^fa
    const int *pos_dev;            // position of the token (device cell), or nullptr: pos_bound is the position
    long long pos_bound;
    int64_t *x;                    // residual row [d]: input of the first block, output of the last
    int64_t *qkv;                  // scratch [(H + 2 Hkv) * hd]
    int64_t *logits;               // scratch [E]
    int8_t *gul;                   // scratch [k][8][eff]: digit planes of silu(gate) * up of the routed experts
    long long *hmax;               // scratch [2][H] row maxima, by block parity
    unsigned long long *Z;         // scratch [2][H] normalisers
    long long *acc;                // scratch [2][H * hd] probability-value sums
    unsigned *bars;                // scratch [6] arrival counters (zeroed by the launcher)
    int *ids_out;                  // optional [n_layers][k]: routed experts of every block
    int64_t *gates_out;            // optional [n_layers][k]
    int *flags;                    // bit 0 digit envelope, 1 RMSNorm envelope, 2 K/V beyond int32, 3 a wait gave up,
                                   // 4 position beyond the bound, 5 a query value beyond int32
    long long inv_sqrt, log2e, clip, sig_log2e, sig_clip;
};
bool decode_shape_ok(int d, int H, int Hkv, int hd, int E, int k, int eff, int down_q);
int decode_max_ctas(int d, int H, int Hkv, int hd, int E, int eff);      // CTAs of one cooperative launch (0: unavailable)
long long decode_key_capacity(int n_ctas, int Hkv, int hd);             // cached keys per KV head one launch can hold
cudaError_t launch_decode(const DecodeArgs &a, int n_ctas, cudaStream_t s);

// Q1_0 linear (q1.cu).  Units: 16-row tiles x 128-weight blocks, 256 B of sign bits in MMA order + 16 scales.
size_t q1_unit_bytes(bool sc32);
cudaError_t launch_q1_repack(const uint8_t *bits, const void *scale, int src_bits, bool sc32, long long out_f, long long nb,
                             uint8_t *units, cudaStream_t s);
cudaError_t launch_q1_prep(const int64_t *x, long long T, long long nb, int8_t *planes, int64_t *totals, int *nl_out,
                           cudaStream_t s);
cudaError_t launch_q1_apply(const uint8_t *units, bool sc32, long long out_f, long long nb, const int8_t *planes,
                            const int64_t *totals, long long T, long long frac, int64_t *out, cudaStream_t s,
                            const int64_t *add = nullptr);
cudaError_t launch_q1_prep_swiglu(const int64_t *gate, const int64_t *up, long long ld, int frac, long long T, long long nb,
                                  int8_t *planes, int64_t *totals, cudaStream_t s);
cudaError_t launch_rmsnorm_pair(const int64_t *x, long long rows_a, long long rows_b, long long width, const int64_t *gain_a,
                                const int64_t *gain_b, int fa, unsigned long long eps, int64_t *out, int *flags, cudaStream_t s);
bool attn_shape_ok(int n_heads, int n_kv, int head_dim);      // shapes launch_attn_decode accepts
void set_q1_stream(int on);        // 1: single-token Q1_0 products through the bulk-copy kernel, 0 (default): per-lane loads
int *shared_flag_word();           // the library's device flag word (bit 1: RMSNorm envelope), NULL without a device
void restore_flag_bits(int bits);  // OR bits back into the flag word (flags an entry set aside while it ran)
cudaError_t launch_q1_silu_mul(const int64_t *gate, const int64_t *up, long long n, int frac, int64_t *out, cudaStream_t s);
cudaError_t launch_q1_embed_row(const uint8_t *units, bool sc32, long long nb, const int *row_dev, long long row_host, int64_t *out,
                                cudaStream_t s);

}  // namespace iie
