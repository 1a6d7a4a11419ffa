/* CPU oracle (C restatement) for the integer MoE block.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker and the timed CPU baseline, never the product.  It restates the
 * reference project's CPU integer path in plain C with OpenMP so that large shapes finish in
 * seconds.  It is validated against the reference's own C kernel (when that is built beside it)
 * and against the NumPy oracle by the CPU test-suite.
 *
 * Reference anchors (paths inside the reference project):
 *   north-mini-code/tools/nmc_qk_kernel.c:16-39   half -> fixed conversion
 *   north-mini-code/tools/nmc_qk_kernel.c:42-82   Q4_K / Q6_K block decode
 *   north-mini-code/tools/nmc_qk_kernel.c:85-120  fused linear, one floor after the full-K sum
 *   north-mini-code/src/nmc/_bonsai/fixedpoint.py:74-96,136-163   exp2 / sigmoid
 *   north-mini-code/src/nmc/cohere2.py:109-111,162-188           silu, top-k, MoE layer
 *   north-mini-code/src/nmc/engine.py:429-443     CPU composition of the MoE block
 *   bonsai/tools/bonsai_q1_kernel.c:85-106        Q1_0 element (per-block floor, modulo 2^64)
 *
 * The linear is written in factored form: per sub-block the code sums q*x and x once and applies
 * the sub-block scale and minimum afterwards.  In exact arithmetic this equals the reference's
 * per-weight form; all sums are kept in 128 bits.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef __int128 i128;

int64_t orc_half_to_fixed(uint16_t h, int frac) {
    int64_t sign = (h >> 15) & 1, e = (h >> 10) & 0x1F, m = h & 0x3FF;
    if (e == 0) e = -24; else { m |= 0x400; e -= 25; }
    e += frac;
    int64_t v;
    if (e >= 0) v = (int64_t)((uint64_t)m << e);
    else {
        int s = (int)(-e); if (s > 40) s = 40;
        int64_t q = m >> s, rem = m & (((int64_t)1 << s) - 1), half = (int64_t)1 << (s - 1);
        v = q + ((rem > half) || (rem == half && (q & 1)));
    }
    return sign ? -v : v;
}

static inline i128 dot_block_q4k(const uint8_t *blk, const int64_t *x, int fw) {
    uint16_t hd, hm; memcpy(&hd, blk, 2); memcpy(&hm, blk + 2, 2);
    const int64_t dq = orc_half_to_fixed(hd, fw), dmq = orc_half_to_fixed(hm, fw);
    const uint8_t *s = blk + 4, *qs = blk + 16;
    i128 acc = 0;
    for (int j = 0; j < 8; j++) {
        int sc, mn;
        if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
        else { sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
        const uint8_t *qb = qs + 32 * (j >> 1);
        const int64_t *xb = x + 32 * j;
        const int sh = (j & 1) ? 4 : 0;
        i128 sq = 0, sx = 0;
        for (int l = 0; l < 32; l++) { sq += (i128)((qb[l] >> sh) & 0xF) * xb[l]; sx += xb[l]; }
        acc += (i128)(dq * sc) * sq - (i128)(dmq * mn) * sx;
    }
    return acc;
}

static inline i128 dot_block_q6k(const uint8_t *blk, const int64_t *x, int fw) {
    const uint8_t *ql = blk, *qh = blk + 128; const int8_t *sc = (const int8_t *)(blk + 192);
    uint16_t hd; memcpy(&hd, blk + 208, 2);
    const int64_t dq = orc_half_to_fixed(hd, fw);
    i128 acc = 0;
    for (int sb = 0; sb < 16; sb++) {           /* sub-block sb covers weights 16*sb .. 16*sb+15 */
        const int half = sb >> 3, k = (sb >> 1) & 3, l0 = (sb & 1) * 16;
        const uint8_t *qlp = ql + 64 * half + 32 * (k & 1) + l0, *qhp = qh + 32 * half + l0;
        const int64_t *xb = x + 16 * sb;
        i128 sq = 0;
        for (int l = 0; l < 16; l++) {
            int nib = (k < 2) ? (qlp[l] & 0xF) : (qlp[l] >> 4);
            int q = (nib | (((qhp[l] >> (2 * k)) & 3) << 4)) - 32;
            sq += (i128)q * xb[l];
        }
        acc += (i128)(dq * sc[8 * half + 2 * k + (sb & 1)]) * sq;
    }
    return acc;
}

/* out[t*out_f+o] = floor(sum_i W[o,i]*x[t,i] / 2^fw); qtype 0 = Q4_K, 1 = Q6_K. */
void orc_qk_linear(const uint8_t *W, const int64_t *x, int64_t T, int64_t out_f, int64_t n_blocks,
                   int fw, int qtype, int64_t *out) {
    const int64_t bs = qtype == 0 ? 144 : 210, in_f = n_blocks * 256;
    #pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < out_f; o++) {
        const uint8_t *row = W + (size_t)o * n_blocks * bs;
        for (int64_t t = 0; t < T; t++) {
            i128 acc = 0;
            for (int64_t b = 0; b < n_blocks; b++)
                acc += qtype == 0 ? dot_block_q4k(row + b * 144, x + t * in_f + b * 256, fw)
                                  : dot_block_q6k(row + b * 210, x + t * in_f + b * 256, fw);
            out[t * out_f + o] = (int64_t)(acc >> fw);
        }
    }
}

static inline int64_t exp2_neg(int64_t u, int fa) {
    static const int64_t C[4] = {65536, 45426, 15743, 3638};
    int64_t c[4]; int s = 16 - fa;
    for (int i = 0; i < 4; i++) c[i] = s >= 0 ? (C[i] >> s) : (C[i] << -s);
    int64_t k = u >> fa, f = u & (((int64_t)1 << fa) - 1);
    int64_t f2 = (f * f) >> fa, f3 = (f2 * f) >> fa;
    int64_t p = c[0] - ((c[1] * f) >> fa) + ((c[2] * f2) >> fa) - ((c[3] * f3) >> fa);
    if (p < 0) p = 0;
    return p >> (k < 63 ? k : 63);
}

int64_t orc_sigmoid(int64_t x, int fa) {
    int s = 16 - fa;
    int64_t log2e = s >= 0 ? (94548 >> s) : ((int64_t)94548 << -s);
    int64_t clip = (((int64_t)(fa + 2)) << (2 * fa)) / log2e;
    int64_t m = x > 0 ? x : 0;
    int64_t d0 = m < clip ? m : clip;
    /* NumPy evaluates m - x and d * log2e in wrapping int64 (only x = INT64_MIN wraps); do the same */
    int64_t d1 = (int64_t)((uint64_t)m - (uint64_t)x);
    if (d1 > clip) d1 = clip;
    int64_t e0 = exp2_neg((d0 * log2e) >> fa, fa);
    int64_t e1 = exp2_neg((int64_t)((uint64_t)d1 * (uint64_t)log2e) >> fa, fa);
    int64_t z = e0 + e1;
    return z == 0 ? 0 : (int64_t)(((i128)e1 << fa) / z);
}

void orc_sigmoid_vec(const int64_t *x, int64_t n, int fa, int64_t *out) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_sigmoid(x[i], fa);
}

static inline int64_t silu1(int64_t x, int fa) { return (int64_t)(((i128)x * orc_sigmoid(x, fa)) >> fa); }

void orc_silu_vec(const int64_t *x, int64_t n, int fa, int64_t *out) {
    for (int64_t i = 0; i < n; i++) out[i] = silu1(x[i], fa);
}

/* ids[k]: k largest logits in descending order, lowest index first among equals. */
void orc_topk_lowidx(const int64_t *logits, int n, int k, int32_t *ids) {
    for (int r = 0; r < k; r++) {
        int best = -1;
        for (int e = 0; e < n; e++) {
            int taken = 0;
            for (int j = 0; j < r; j++) if (ids[j] == e) { taken = 1; break; }
            if (!taken && (best < 0 || logits[e] > logits[best])) best = e;
        }
        ids[r] = best;
    }
}

/* The MoE FFN on T tokens, composed the way the reference engine's CPU branch composes it:
 * router linear, top-k, sigmoid gates, then per (token, selected expert) gate/up linears, integer
 * SiLU, product, down linear, one floor of (down * gate) per expert, and an exact sum.
 * Weight tables hold n_experts raw tensors each; qtypes apply to all experts of a projection.
 * scratch must hold T*n_experts + 2*e_ffn + d_model int64. */
void orc_moe_block(const uint8_t *router, int router_qtype, const uint8_t *const *gate,
                   const uint8_t *const *up, const uint8_t *const *down, int gate_qtype, int down_qtype,
                   int n_experts, int k, const int64_t *h, int64_t T, int64_t d_model, int64_t e_ffn,
                   int fa, int fw, int32_t *ids_out, int64_t *gates_out, int64_t *out, int64_t *scratch) {
    const int64_t nb_in = d_model / 256, nb_dn = e_ffn / 256;
    int64_t *logits = scratch, *g = logits + T * n_experts, *u = g + e_ffn, *dn = u + e_ffn;
    orc_qk_linear(router, h, T, n_experts, nb_in, fw, router_qtype, logits);
    for (int64_t t = 0; t < T; t++) {
        int32_t *ids = ids_out + t * k; int64_t *gw = gates_out + t * k;
        orc_topk_lowidx(logits + t * n_experts, n_experts, k, ids);
        for (int j = 0; j < k; j++) gw[j] = orc_sigmoid(logits[t * n_experts + ids[j]], fa);
        for (int64_t o = 0; o < d_model; o++) out[t * d_model + o] = 0;
        for (int j = 0; j < k; j++) {
            const int e = ids[j];
            orc_qk_linear(gate[e], h + t * d_model, 1, e_ffn, nb_in, fw, gate_qtype, g);
            orc_qk_linear(up[e], h + t * d_model, 1, e_ffn, nb_in, fw, gate_qtype, u);
            for (int64_t i = 0; i < e_ffn; i++) g[i] = (int64_t)(((i128)silu1(g[i], fa) * u[i]) >> fa);
            orc_qk_linear(down[e], g, 1, d_model, nb_dn, fw, down_qtype, dn);
            for (int64_t o = 0; o < d_model; o++)
                out[t * d_model + o] = (int64_t)((uint64_t)out[t * d_model + o] +
                                                 (uint64_t)(int64_t)(((i128)dn[o] * gw[j]) >> fa));
        }
    }
}

static inline int64_t arshift64(int64_t v, int s) { return s <= 0 ? v : (s >= 63 ? (v < 0 ? -1 : 0) : (v >> s)); }

/* Q1_0 linear: out[t,o] = sum_b arshift((sum_i sign_i x_i) * scale[o,b], frac), all modulo 2^64.
 * bits: [out_f][n_blocks][16], bit i of byte j (LSB first) is weight 8j+i, set bit = +1. */
void orc_q1_linear(const int64_t *x, const uint8_t *bits, const int64_t *scale, int64_t T, int64_t out_f,
                   int64_t n_blocks, int frac, int64_t *out) {
    #pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < out_f; o++) {
        for (int64_t t = 0; t < T; t++) {
            uint64_t total = 0;
            for (int64_t b = 0; b < n_blocks; b++) {
                const uint8_t *bb = bits + ((size_t)o * n_blocks + b) * 16;
                const int64_t *xb = x + (t * n_blocks + b) * 128;
                uint64_t ssum = 0;
                for (int i = 0; i < 128; i++)
                    ssum += ((bb[i >> 3] >> (i & 7)) & 1) ? (uint64_t)xb[i] : (uint64_t)0 - (uint64_t)xb[i];
                uint64_t prod = ssum * (uint64_t)scale[o * n_blocks + b];
                total += (uint64_t)arshift64((int64_t)prod, frac);
            }
            out[t * out_f + o] = (int64_t)total;
        }
    }
}

int orc_available(void) { return 0; }
