// Prefill attention by query tiles: the three passes of the exact softmax (north-mini-code/src/nmc/cohere2.py:324-354 with
// _bonsai/fixedpoint.py:99-133; the arithmetic is stated at the top of attn.cu) for `batch` consecutive tokens of one
// sequence, sixteen tokens x the query heads of one KV head per CTA.
//
// The per-token kernels of attn.cu stage a 64-key chunk of K (or V) for the eight score columns of ONE token; here the chunk
// is staged once for 128 (token, head) rows, as byte planes, and both products run on the tensor cores with the byte
// decomposition of attn_fat_kernel: an int32 is b0 + 2^8 b1 + 2^16 b2 + 2^24 b3 with b0..b2 unsigned and b3 signed, every
// byte pair is an exact int8 MMA, pairs of equal a + b share an int32 accumulator, and the 64-bit value is re-assembled as
// sum_s 256^s acc_s in wrapping arithmetic (which is what the reference's int64 products do).  Where every value of an
// operand lies in [-2^23, 2^23) its top byte plane is left out (three planes, the third signed), decided per chunk.
// Two forms of each product: tcgen05 (kind::i8, M 128, accumulators in TMEM; the default) and mma.sync m16n8k32 (64-bit sums
// in registers; for key spans the int32 TMEM accumulators of the probability x value pass do not carry, and as the partner
// the tests compare against).  The exponentials in between run one warp per (token, head) row and leave probabilities.
// Causality and the window are masks per (token, key); a masked probability is zero.  A query beyond int32 (the reference
// multiplies it as int64) takes a scalar path inside the scores kernels.
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace iie {

namespace {

constexpr int PT_Q = 16;                    // tokens of a tile
constexpr int PT_HEADS = 8;                 // query heads of a KV head (rows beyond the real count are zero)
constexpr int PT_COLS = PT_Q * PT_HEADS;    // 128 (token, head) columns / rows
constexpr int PT_THREADS = 512;
constexpr int PT_CH = 64;                   // keys per chunk
constexpr int PT_WALK = 4;                  // chunks a scores CTA walks
constexpr int PT_PLD = PT_CH + 16;          // bytes per row of a key-major byte plane (probabilities, transposed values)

// D(16x8,s32) += A(16x32, 8-bit, row) * B(32x8, 8-bit, col), signedness per operand
template <bool A_SIGNED, bool B_SIGNED>
__device__ __forceinline__ void pt_mma(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (A_SIGNED && B_SIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else if (A_SIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else if (B_SIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// four int32 -> one word per byte plane (byte i of plane b = byte b of value i)
__device__ __forceinline__ void pt_planes(uint32_t x, uint32_t y, uint32_t z, uint32_t w, uint32_t &d0, uint32_t &d1, uint32_t &d2, uint32_t &d3) {
    const uint32_t t0 = __byte_perm(x, y, 0x5140), t1 = __byte_perm(x, y, 0x7362);
    const uint32_t t2 = __byte_perm(z, w, 0x5140), t3 = __byte_perm(z, w, 0x7362);
    d0 = __byte_perm(t0, t2, 0x5410); d1 = __byte_perm(t0, t2, 0x7632);
    d2 = __byte_perm(t1, t3, 0x5410); d3 = __byte_perm(t1, t3, 0x7632);
}

__device__ __forceinline__ void pt_rotate(const AttnArgs &a, long long pos, int i, int64_t &x0, int64_t &x1) {
    if (!a.rope) return;
    const int half = a.hd / 2;
    const int64_t c = a.cos[pos * half + i], s = a.sin[pos * half + i];
    const int64_t y0 = (x0 * c - x1 * s) >> a.fa, y1 = (x0 * s + x1 * c) >> a.fa;
    x0 = y0; x1 = y1;
}

struct Tile {                               // the sixteen tokens of a CTA
    long long t0, pos0, pos_last, lo_t;
    int nq;
};
__device__ __forceinline__ Tile pt_tile(const AttnArgs &a, long long tile) {
    Tile t;
    t.t0 = tile * PT_Q;
    t.nq = (int)min((long long)PT_Q, (long long)a.batch - t.t0);
    t.pos0 = a.pos + t.t0;
    t.pos_last = t.pos0 + t.nq - 1;
    t.lo_t = (a.window > 0 && t.pos0 - a.window + 1 > 0) ? t.pos0 - a.window + 1 : 0;      // first key the first token sees
    return t;
}
__device__ __forceinline__ long long pt_lo(const AttnArgs &a, long long pos) { return (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0; }

// ---- pass 1: scores[token][head][key] and the row maxima ----------------------------------------------------------------
// grid (walks, Hkv, tiles): CTA x walks PT_WALK chunks of the tile's key span.  16 warps = 4 key tiles x 4 groups of four
// tokens; a warp multiplies one key tile with two tokens at a time (56 accumulator registers).
template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1) attn_tile_scores_kernel(const AttnArgs a) {
    constexpr int QLD = HD + 16, HALF = HD / 2, VPT = HD / 32;     // bytes per plane row; 16-byte vectors of a chunk per thread
    extern __shared__ __align__(16) unsigned char pt_smem[];
    __shared__ long long s_max[PT_COLS];
    __shared__ int s_wide, s_qwide24;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rep = a.H / a.Hkv, kv = blockIdx.y;
    const Tile T = pt_tile(a, (long long)gridDim.z - 1 - blockIdx.z);           // long tiles first
    const long long c_first = T.lo_t / PT_CH + (long long)blockIdx.x * PT_WALK;
    if (c_first * PT_CH > T.pos_last) return;
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    int8_t *qd = reinterpret_cast<int8_t *>(pt_smem);             // query byte planes [4][128 columns][QLD], column = token * 8 + head
    int8_t *kd = qd + 4 * PT_COLS * QLD;                          // key byte planes [2 buffers][4][64 keys][QLD]
    if (tid < PT_COLS) s_max[tid] = INT64_MIN;
    if (tid == 0) { s_wide = 0; s_qwide24 = 0; }
    __syncthreads();
    bool wide = false, wide24 = false;
    for (int idx = tid; idx < PT_COLS * HALF; idx += PT_THREADS) {
        const int col = idx / HALF, i = idx - col * HALF, qi = col >> 3, h = col & 7;
        const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + HALF : 2 * i + 1;
        int64_t x0 = 0, x1 = 0;
        if (qi < T.nq && h < rep) {
            const int64_t *src = a.q + ((T.t0 + qi) * a.H + kv * rep + h) * HD;
            x0 = src[i0]; x1 = src[i1];
            pt_rotate(a, T.pos0 + qi, i, x0, x1);
        }
#pragma unroll
        for (int b = 0; b < 4; b++) {
            qd[(b * PT_COLS + col) * QLD + i0] = (int8_t)((uint32_t)(int32_t)x0 >> (8 * b));
            qd[(b * PT_COLS + col) * QLD + i1] = (int8_t)((uint32_t)(int32_t)x1 >> (8 * b));
        }
        wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
        wide24 |= x0 < -(1 << 23) || x0 >= (1 << 23) || x1 < -(1 << 23) || x1 >= (1 << 23);
    }
    if (wide) s_wide = 1;
    if (wide24) s_qwide24 = 1;
    __syncthreads();
    auto publish_max = [&]() {
        __syncthreads();
        if (tid < PT_COLS && s_max[tid] != INT64_MIN) {
            const int qi = tid >> 3, h = tid & 7;
            atomicMax(a.hmax + (T.t0 + qi) * a.H + kv * rep + h, s_max[tid]);
        }
    };
    if (s_wide) {
        // a query value beyond int32: 64-bit wrapping products, one thread per (key, column); the rotated queries as int64
        // take the place of every byte plane
        long long *q64 = reinterpret_cast<long long *>(pt_smem);   // [128][HD]
        for (int idx = tid; idx < PT_COLS * HALF; idx += PT_THREADS) {
            const int col = idx / HALF, i = idx - col * HALF, qi = col >> 3, h = col & 7;
            const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + HALF : 2 * i + 1;
            int64_t x0 = 0, x1 = 0;
            if (qi < T.nq && h < rep) {
                const int64_t *src = a.q + ((T.t0 + qi) * a.H + kv * rep + h) * HD;
                x0 = src[i0]; x1 = src[i1];
                pt_rotate(a, T.pos0 + qi, i, x0, x1);
            }
            q64[col * HD + i0] = x0; q64[col * HD + i1] = x1;
        }
        __syncthreads();
        for (int w = 0; w < PT_WALK; w++) {
            const long long l0 = (c_first + w) * PT_CH;
            if (l0 > T.pos_last) break;
            for (int idx = tid; idx < PT_CH * PT_COLS; idx += PT_THREADS) {
                const int key = idx >> 7, col = idx & 127, qi = col >> 3, h = col & 7;
                const long long l = l0 + key, pos_q = T.pos0 + qi;
                if (qi >= T.nq || h >= rep || l > pos_q || l < pt_lo(a, pos_q)) continue;
                const int32_t *kk = a.kcache + ((long long)kv * a.Lmax + l) * HD;
                long long dot = 0;
                for (int j = 0; j < HD; j++) dot += q64[col * HD + j] * (long long)kk[j];
                const long long sc = ((dot >> a.fa) * a.inv_sqrt) >> a.fa;
                a.scores[((T.t0 + qi) * a.H + kv * rep + h) * Ls + l] = sc;
                atomicMax(&s_max[col], sc);
            }
        }
        publish_max();
        return;
    }
    int4 kreg[VPT];
    auto load = [&](long long c) {                                 // keys of chunk c into registers (rows past the last token: zero)
#pragma unroll
        for (int u = 0; u < VPT; u++) {
            const int v = tid + u * PT_THREADS, key = v / (HD / 4), part = v - key * (HD / 4);
            const long long l = c * PT_CH + key;
            kreg[u] = l <= T.pos_last ? __ldg(reinterpret_cast<const int4 *>(a.kcache + ((long long)kv * a.Lmax + l) * HD) + part) : make_int4(0, 0, 0, 0);
        }
    };
    auto store = [&](int buf) {                                    // registers -> byte planes of buffer buf; true if every key value fits 24 bits
        bool fits = true;
#pragma unroll
        for (int u = 0; u < VPT; u++) {
            const int v = tid + u * PT_THREADS, key = v / (HD / 4), part = v - key * (HD / 4);
            const int vals[4] = {kreg[u].x, kreg[u].y, kreg[u].z, kreg[u].w};
#pragma unroll
            for (int i = 0; i < 4; i++) fits &= vals[i] >= -(1 << 23) && vals[i] < (1 << 23);
            uint32_t d[4];
            pt_planes((uint32_t)kreg[u].x, (uint32_t)kreg[u].y, (uint32_t)kreg[u].z, (uint32_t)kreg[u].w, d[0], d[1], d[2], d[3]);
#pragma unroll
            for (int b = 0; b < 4; b++) *reinterpret_cast<uint32_t *>(kd + ((buf * 4 + b) * PT_CH + key) * QLD + part * 4) = d[b];
        }
        return fits;
    };
    const int mt = warp & 3, ng = warp >> 2;
    const bool q_narrow = s_qwide24 == 0;
    load(c_first);
    for (int w = 0; w < PT_WALK; w++) {
        const long long c = c_first + w, l0 = c * PT_CH;
        if (l0 > T.pos_last) break;                                // uniform over the CTA
        const int buf = w & 1;
        const bool k_fits = store(buf);
        const bool narrow = __syncthreads_and(k_fits) && q_narrow;   // planes of chunk c visible; the other buffer's readers are done
        if (w + 1 < PT_WALK && l0 + PT_CH <= T.pos_last) load(c + 1);
        const long long key_lo = l0 + mt * 16, key_hi = key_lo + 15;
        auto tile_pairs = [&](auto nb_c) {                        // NB byte planes per operand, the last one signed
        constexpr int NB = decltype(nb_c)::value;
#pragma unroll 1
        for (int np = 0; np < 2; np++) {
            const int n0 = ng * 4 + np * 2;                        // tokens n0 and n0 + 1
            // nothing of this key tile is visible to either token: warp-uniform skip
            if (n0 >= T.nq || key_lo > T.pos0 + n0 + 1 || key_hi < pt_lo(a, T.pos0 + n0)) continue;
            int acc[2][2 * NB - 1][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int s = 0; s < 2 * NB - 1; s++) { acc[j][s][0] = acc[j][s][1] = acc[j][s][2] = acc[j][s][3] = 0; }
#pragma unroll
            for (int st = 0; st < HD / 32; st++) {
                uint32_t A[NB][4];
#pragma unroll
                for (int aa = 0; aa < NB; aa++) {
                    const int8_t *base = kd + ((buf * 4 + aa) * PT_CH + mt * 16 + g) * QLD + 32 * st + 4 * t;
                    A[aa][0] = *reinterpret_cast<const uint32_t *>(base); A[aa][1] = *reinterpret_cast<const uint32_t *>(base + 8 * QLD);
                    A[aa][2] = *reinterpret_cast<const uint32_t *>(base + 16); A[aa][3] = *reinterpret_cast<const uint32_t *>(base + 8 * QLD + 16);
                }
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const int8_t *qb = qd + (b * PT_COLS + (n0 + j) * 8 + g) * QLD + 32 * st + 4 * t;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(qb), b1 = *reinterpret_cast<const uint32_t *>(qb + 16);
#pragma unroll
                        for (int aa = 0; aa < NB; aa++) {
                            if (aa < NB - 1 && b < NB - 1) pt_mma<false, false>(acc[j][aa + b], A[aa], b0, b1);
                            else if (aa < NB - 1) pt_mma<false, true>(acc[j][aa + b], A[aa], b0, b1);
                            else if (b < NB - 1) pt_mma<true, false>(acc[j][aa + b], A[aa], b0, b1);
                            else pt_mma<true, true>(acc[j][aa + b], A[aa], b0, b1);
                        }
                    }
            }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int qi = n0 + j;
                const long long pos_q = T.pos0 + qi, lo_q = pt_lo(a, pos_q);
                long long m2[2] = {INT64_MIN, INT64_MIN};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    long long dot = 0;
#pragma unroll
                    for (int s = 2 * NB - 2; s >= 0; s--) dot = dot * 256 + (long long)acc[j][s][i];
                    const long long l = key_lo + g + (i >= 2 ? 8 : 0);
                    const int h = 2 * t + (i & 1);
                    if (qi < T.nq && h < rep && l <= pos_q && l >= lo_q) {
                        const long long sc = ((dot >> a.fa) * a.inv_sqrt) >> a.fa;
                        a.scores[((T.t0 + qi) * a.H + kv * rep + h) * Ls + l] = sc;
                        m2[i & 1] = max(m2[i & 1], sc);
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    long long m = m2[u];
                    m = max(m, __shfl_xor_sync(0xffffffffu, m, 4)); m = max(m, __shfl_xor_sync(0xffffffffu, m, 8));
                    m = max(m, __shfl_xor_sync(0xffffffffu, m, 16));
                    if (g == 0 && m != INT64_MIN) atomicMax(&s_max[qi * 8 + 2 * t + u], m);
                }
            }
        }
        };
        if (narrow) tile_pairs(std::integral_constant<int, 3>{}); else tile_pairs(std::integral_constant<int, 4>{});
    }
    publish_max();
}

// ---- pass 2: exponentials, their sum and the probabilities, one warp per (token, head) row ----------------------------------
// e_l = 2^-((min(max - score_l, clip) * log2e) >> fa) for the visible keys of the row, two keys per lane and step; the row
// belongs to this warp, so its normaliser Z needs no atomics and the same lanes turn their e_l into p_l = (e_l << fa) / Z in
// place (through the reciprocal of Z with an exact fix-up: the estimate is at most 2 low).
__global__ void __launch_bounds__(256) attn_tile_exp_kernel(const AttnArgs a) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), n_rows = (long long)a.batch * a.H;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const long long tok = row / a.H, pos = a.pos + tok, lo = pt_lo(a, pos), Ls = a.Ls ? a.Ls : a.Lmax;
    const int64_t *sc = a.scores + row * Ls;
    int32_t *e = a.e + row * Ls;
    const long long m = a.hmax[row];
    unsigned long long sum = 0;
    for (long long l = (lo & ~1LL) + 2 * lane; l <= pos; l += 64) {
        const longlong2 s2 = *reinterpret_cast<const longlong2 *>(sc + l);
        int2 e2 = make_int2(0, 0);
        if (l >= lo) {
            long long d = m - s2.x;
            d = d < a.clip ? d : a.clip;
            e2.x = (int)exp2_neg_fixed((d * a.log2e) >> a.fa, a.fa);
        }
        if (l + 1 <= pos) {
            long long d = m - s2.y;
            d = d < a.clip ? d : a.clip;
            e2.y = (int)exp2_neg_fixed((d * a.log2e) >> a.fa, a.fa);
        }
        sum += (unsigned long long)(unsigned)e2.x + (unsigned long long)(unsigned)e2.y;
        *reinterpret_cast<int2 *>(e + l) = e2;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (lane == 0) a.Z[row] = sum;
    if (sum == 0) return;                                          // (cannot happen: the row maximum has e = 2^fa)
    const unsigned long long inv = 0xFFFFFFFFFFFFFFFFULL / sum;
    auto prob = [&](int ev) {
        const unsigned long long n = (unsigned long long)(unsigned)ev << a.fa;
        unsigned long long q = __umul64hi(n, inv), r = n - q * sum;
        while (r >= sum) { q++; r -= sum; }
        return (int)q;
    };
    for (long long l = (lo & ~1LL) + 2 * lane; l <= pos; l += 64) {
        int2 e2 = *reinterpret_cast<int2 *>(e + l);               // this lane's own stores
        e2.x = prob(e2.x); e2.y = prob(e2.y);
        *reinterpret_cast<int2 *>(e + l) = e2;
    }
}

// ---- pass 3: out[token][head][dim] = (sum over keys of p x v) >> fa --------------------------------------------------------
// grid (1, Hkv, tiles): the CTA walks every chunk of the tile's key span.  Rows are head * 16 + token; 16 warps = 8 heads x
// the two halves of the head dimension; the 64-bit sums of a thread's outputs stay in registers over the whole walk.
template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1) attn_tile_pv_kernel(const AttnArgs a) {
    constexpr int NT = HD / 16;                                    // 8-wide dimension tiles of a warp
    constexpr int VU = HD / 32;                                    // (dimension, four keys) units of a thread per chunk
    extern __shared__ __align__(16) unsigned char pt_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rep = a.H / a.Hkv, kv = blockIdx.y;
    const Tile T = pt_tile(a, (long long)gridDim.z - 1 - blockIdx.z);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    uint8_t *vT = pt_smem;                                         // value byte planes [4][HD dims][PT_PLD], keys along a row
    uint8_t *pT = vT + 4 * HD * PT_PLD;                            // probability byte planes [3][128 rows][PT_PLD]
    int32_t *vraw = reinterpret_cast<int32_t *>(pT + 3 * PT_COLS * PT_PLD);      // the next chunk's values as they lie in the cache [64][HD]
    auto fetch_v = [&](long long c) {                              // asynchronous copies, no registers held (rows past the last token: zero)
#pragma unroll
        for (int u = 0; u < VU; u++) {
            const int v = tid + u * PT_THREADS, key = v / (HD / 4), part = v - key * (HD / 4);
            const long long l = c * PT_CH + key;
            int32_t *dst = vraw + key * HD + part * 4;
            if (l <= T.pos_last) {
                const int32_t *src = a.vcache + ((long long)kv * a.Lmax + l) * HD + part * 4;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
            } else *reinterpret_cast<int4 *>(dst) = make_int4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int vd = tid % HD, vq0 = tid / HD;                       // this thread's dimension and first key group of the transposition
    auto convert_v = [&]() {                                       // raw chunk -> transposed byte planes; true if every value fits 24 bits
        bool fits = true;
#pragma unroll
        for (int u = 0; u < VU; u++) {
            const int kq = vq0 + u * (PT_THREADS / HD);
            int x[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { x[i] = vraw[(4 * kq + i) * HD + vd]; fits &= x[i] >= -(1 << 23) && x[i] < (1 << 23); }
            uint32_t d[4];
            pt_planes((uint32_t)x[0], (uint32_t)x[1], (uint32_t)x[2], (uint32_t)x[3], d[0], d[1], d[2], d[3]);
#pragma unroll
            for (int b = 0; b < 4; b++) *reinterpret_cast<uint32_t *>(vT + (b * HD + vd) * PT_PLD + 4 * kq) = d[b];
        }
        return fits;
    };
    long long acc64[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { acc64[nt][0] = acc64[nt][1] = acc64[nt][2] = acc64[nt][3] = 0; }
    const int mt = warp & 7, nh = warp >> 3;
    const long long c_lo = T.lo_t / PT_CH, c_hi = T.pos_last / PT_CH;
    fetch_v(c_lo);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                               // the first chunk's values
    for (long long c = c_lo; c <= c_hi; c++) {
        const long long l0 = c * PT_CH;
        // probabilities of this chunk: requested first, the value planes are transposed while they arrive
        int4 e4[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int row = (tid >> 4) + 32 * u, kg = tid & 15, h = row >> 4, qi = row & 15;
            e4[u] = make_int4(0, 0, 0, 0);
            if (qi < T.nq && h < rep && l0 + 4 * kg <= T.pos0 + qi)
                e4[u] = __ldg(reinterpret_cast<const int4 *>(a.e + ((T.t0 + qi) * a.H + kv * rep + h) * Ls + l0 + 4 * kg));
        }
        const bool v_fits = convert_v();
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int row = (tid >> 4) + 32 * u, kg = tid & 15, qi = row & 15;
            const long long pos_q = T.pos0 + qi, lo_q = pt_lo(a, pos_q);
            const int ev[4] = {e4[u].x, e4[u].y, e4[u].z, e4[u].w};
            uint32_t p[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const long long l = l0 + 4 * kg + i;
                uint32_t pv = 0;
                if (l <= pos_q && l >= lo_q) pv = (uint32_t)ev[i];
                p[i] = pv;
            }
            uint32_t d0, d1, d2, d3;
            pt_planes(p[0], p[1], p[2], p[3], d0, d1, d2, d3);
            uint8_t *dst = pT + row * PT_PLD + 4 * kg;
            *reinterpret_cast<uint32_t *>(dst) = d0;
            *reinterpret_cast<uint32_t *>(dst + PT_COLS * PT_PLD) = d1;
            *reinterpret_cast<uint32_t *>(dst + 2 * PT_COLS * PT_PLD) = d2;
        }
        const bool narrow = __syncthreads_and(v_fits);             // planes of chunk c visible, the raw buffer is free
        if (c < c_hi) fetch_v(c + 1);
        // the head's sixteen tokens x this warp's dimensions; tokens that see nothing of the chunk have zero probabilities
        uint32_t A[2][3][4];
#pragma unroll
        for (int ks = 0; ks < 2; ks++)
#pragma unroll
            for (int b = 0; b < 3; b++) {
                const uint8_t *base = pT + (b * PT_COLS + mt * 16 + g) * PT_PLD + 32 * ks + 4 * t;
                A[ks][b][0] = *reinterpret_cast<const uint32_t *>(base); A[ks][b][1] = *reinterpret_cast<const uint32_t *>(base + 8 * PT_PLD);
                A[ks][b][2] = *reinterpret_cast<const uint32_t *>(base + 16); A[ks][b][3] = *reinterpret_cast<const uint32_t *>(base + 8 * PT_PLD + 16);
            }
        auto dims = [&](auto nb_c) {                               // NBV value planes, the last one signed
        constexpr int NBV = decltype(nb_c)::value;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            int acc[NBV + 2][4];
#pragma unroll
            for (int s = 0; s < NBV + 2; s++) { acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0; }
            const int dim0 = (nh * NT + nt) * 8;
#pragma unroll
            for (int ks = 0; ks < 2; ks++)
#pragma unroll
                for (int b = 0; b < NBV; b++) {
                    const uint8_t *bp = vT + (b * HD + dim0 + g) * PT_PLD + 32 * ks + 4 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp), b1 = *reinterpret_cast<const uint32_t *>(bp + 16);
#pragma unroll
                    for (int aa = 0; aa < 3; aa++) {
                        if (b < NBV - 1) pt_mma<false, false>(acc[aa + b], A[ks][aa], b0, b1);
                        else pt_mma<false, true>(acc[aa + b], A[ks][aa], b0, b1);
                    }
                }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                long long s64 = 0;
#pragma unroll
                for (int s = NBV + 1; s >= 0; s--) s64 = s64 * 256 + (long long)acc[s][i];
                acc64[nt][i] += s64;
            }
        }
        };
        if (narrow) dims(std::integral_constant<int, 3>{}); else dims(std::integral_constant<int, 4>{});
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                           // the planes may be overwritten; the next chunk's values have landed
    }
    if (mt < rep) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int qi = g + (i >= 2 ? 8 : 0), dim = (nh * NT + nt) * 8 + 2 * t + (i & 1);
                if (qi < T.nq) a.out[((T.t0 + qi) * a.H + kv * rep + mt) * HD + dim] = acc64[nt][i] >> a.fa;
            }
    }
}


// ---- pass 3 on the 5th-generation tensor cores ---------------------------------------------------------------------------
// D[row = head * 16 + token][dim] over a 64-dimension half of the head: grid (HD / 64, Hkv, tiles).  The probability byte
// planes (A, 128 rows x 64 keys) and the transposed value byte planes (B, 64 dims x 64 keys) of a chunk are written by sixteen
// producer warps into the canonical K-major shared-memory layout (8 x 16-byte core matrices, no swizzle), three stages deep;
// one thread issues tcgen05.mma kind::i8 (M 128, N 64, K 32), one per byte pair and K step, pairs of equal a + b into the
// same TMEM accumulator.  The int32 accumulators run over the WHOLE key span (at most 3 pairs x 255^2 x 64 keys per chunk
// and accumulator, so up to 170 chunks stay below 2^31: the launcher bounds the span), and are read out once at the end:
// sum_s 256^s acc_s in wrapping 64-bit arithmetic, shifted, stored.  Every wait is bounded; on a time-out the CTA raises flag
// bit 3, leaves its loops, frees its TMEM and exits.
constexpr int PC_PRODUCERS = 512, PC_THREADS = PC_PRODUCERS + 32, PC_STAGES = 3, PC_N = 64;
constexpr int PC_P_PLANE = PT_COLS * PT_CH, PC_V_PLANE = PC_N * PT_CH;             // 8192 / 4096 bytes
constexpr int PC_STAGE = 3 * PC_P_PLANE + 4 * PC_V_PLANE;                          // 40960 bytes
constexpr unsigned PC_WAIT_LIMIT = 1u << 24;
constexpr long long PC_MAX_CHUNKS = 160;

__device__ __forceinline__ uint32_t pc_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pc_wait(uint64_t *b, uint32_t parity, volatile int *abort_flag) {
    for (unsigned it = 0; it < PC_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(pc_u32(b)), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// K-major, no swizzle: LBO = distance of the two 16-byte K halves of one MMA, SBO = distance of consecutive 8-row groups
__device__ __forceinline__ uint64_t pc_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}
__device__ __forceinline__ void pc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void pc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pc_u32(bar)) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(PC_THREADS, 1) attn_tile_pv_tc_kernel(const AttnArgs a) {
    extern __shared__ __align__(1024) unsigned char pc_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(pc_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[PC_STAGES], empty_bar[PC_STAGES], accum_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rep = a.H / a.Hkv, kv = blockIdx.y, dim_base = blockIdx.x * PC_N;
    const Tile T = pt_tile(a, (long long)gridDim.z - 1 - blockIdx.z);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    const long long c_lo = T.lo_t / PT_CH, c_hi = T.pos_last / PT_CH;
    const int n_chunks = (int)(c_hi - c_lo + 1);
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < PC_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&full_bar[s])), "r"(PC_PRODUCERS / 32));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&empty_bar[s])), "r"(1));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&accum_bar)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PC_PRODUCERS / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pc_u32(&s_tmem)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp < PC_PRODUCERS / 32) {
        // ================= producers: every warp writes whole core matrices (8 rows x 16 bytes), lane = (row, 4-key word) ====
        const int r8 = lane >> 2, w4 = lane & 3;
        for (int ci = 0; ci < n_chunks; ci++) {
            const int s = ci % PC_STAGES;
            if (ci >= PC_STAGES && !pc_wait(&empty_bar[s], ((ci / PC_STAGES) - 1) & 1, &s_abort)) break;
            unsigned char *stage = smem + (size_t)s * PC_STAGE;
            const long long l0 = (c_lo + ci) * PT_CH;
            // probabilities: 16 row groups x 4 key quarters = 64 core matrices per plane, four per warp
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int cm = warp + 16 * u, rg = cm & 15, kq = cm >> 4;
                const int row = rg * 8 + r8, h = row >> 4, qi = row & 15;
                const long long pos_q = T.pos0 + qi, lo_q = pt_lo(a, pos_q), l = l0 + 16 * kq + 4 * w4;
                int4 p4 = make_int4(0, 0, 0, 0);
                if (qi < T.nq && h < rep && l <= pos_q && l + 3 >= lo_q) {
                    p4 = *reinterpret_cast<const int4 *>(a.e + ((T.t0 + qi) * a.H + kv * rep + h) * Ls + l);
                    if (l < lo_q) p4.x = 0;
                    if (l + 1 > pos_q || l + 1 < lo_q) p4.y = 0;
                    if (l + 2 > pos_q || l + 2 < lo_q) p4.z = 0;
                    if (l + 3 > pos_q || l + 3 < lo_q) p4.w = 0;
                }
                uint32_t d0, d1, d2, d3;
                pt_planes((uint32_t)p4.x, (uint32_t)p4.y, (uint32_t)p4.z, (uint32_t)p4.w, d0, d1, d2, d3);
                unsigned char *dst = stage + kq * (PT_COLS * 16) + rg * 128 + r8 * 16 + w4 * 4;
                *reinterpret_cast<uint32_t *>(dst) = d0;
                *reinterpret_cast<uint32_t *>(dst + PC_P_PLANE) = d1;
                *reinterpret_cast<uint32_t *>(dst + 2 * PC_P_PLANE) = d2;
            }
            // values, transposed: 8 dim groups x 4 key quarters = 32 core matrices per plane, two per warp
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int cm = warp + 16 * u, dg = cm & 7, kq = cm >> 3;
                const int dim = dim_base + dg * 8 + r8;
                uint32_t x[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const long long l = l0 + 16 * kq + 4 * w4 + i;
                    x[i] = l <= T.pos_last ? (uint32_t)__ldg(a.vcache + ((long long)kv * a.Lmax + l) * HD + dim) : 0u;
                }
                uint32_t d[4];
                pt_planes(x[0], x[1], x[2], x[3], d[0], d[1], d[2], d[3]);
                unsigned char *dst = stage + 3 * PC_P_PLANE + kq * (PC_N * 16) + dg * 128 + r8 * 16 + w4 * 4;
#pragma unroll
                for (int b = 0; b < 4; b++) *reinterpret_cast<uint32_t *>(dst + b * PC_V_PLANE) = d[b];
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> visible to the MMA
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pc_u32(&full_bar[s])) : "memory");
        }
        // ================= read-out: warps 0..3, TMEM lane = row ==============================================================
        if (warp < 4 && pc_wait(&accum_bar, 0, &s_abort)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = warp * 32 + lane, h = row >> 4, qi = row & 15;
            const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
            int64_t *dst = a.out + ((T.t0 + qi) * a.H + kv * rep + h) * HD + dim_base;
            for (int c0 = 0; c0 < PC_N; c0 += 8) {
                int r[6][8];
#pragma unroll
                for (int s = 0; s < 6; s++)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[s][0]), "=r"(r[s][1]), "=r"(r[s][2]), "=r"(r[s][3]), "=r"(r[s][4]), "=r"(r[s][5]), "=r"(r[s][6]), "=r"(r[s][7])
                                 : "r"(tlane + s * PC_N + c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (qi < T.nq && h < rep) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        long long s64 = 0;
#pragma unroll
                        for (int s = 5; s >= 0; s--) s64 = s64 * 256 + (long long)r[s][j];
                        dst[c0 + j] = s64 >> a.fa;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
        // ================= MMA issuer ===========================================================================================
        if (lane == 0) {
            constexpr uint32_t IDESC_U = (2u << 4) | ((uint32_t)(PC_N >> 3) << 17) | ((uint32_t)(PT_COLS >> 4) << 24);      // u8 x u8 -> s32
            constexpr uint32_t IDESC_S = IDESC_U | (1u << 10);                                                                 // u8 x s8 (top value byte)
            bool ok = true;
            for (int ci = 0; ci < n_chunks && ok; ci++) {
                const int s = ci % PC_STAGES;
                ok = pc_wait(&full_bar[s], (ci / PC_STAGES) & 1, &s_abort);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t stage = pc_u32(smem + (size_t)s * PC_STAGE);
                const uint64_t dp0 = pc_desc(stage, PT_COLS * 16, 128), dv0 = pc_desc(stage + 3 * PC_P_PLANE, PC_N * 16, 128);
                const uint32_t later = ci > 0 ? 1u : 0u;
#pragma unroll
                for (int ks = 0; ks < 2; ks++)
#pragma unroll
                    for (int b = 0; b < 4; b++)
#pragma unroll
                        for (int aa = 0; aa < 3; aa++) {
                            const bool first = ks == 0 && (b == 0 || aa == 2);            // first product into accumulator aa + b
                            const uint64_t dp = dp0 + (uint64_t)((aa * PC_P_PLANE + ks * 2 * PT_COLS * 16) >> 4);
                            const uint64_t dv = dv0 + (uint64_t)((b * PC_V_PLANE + ks * 2 * PC_N * 16) >> 4);
                            pc_mma(tmem + (aa + b) * PC_N, dp, dv, b == 3 ? IDESC_S : IDESC_U, first ? later : 1u);
                        }
                pc_commit(&empty_bar[s]);
            }
            if (ok) pc_commit(&accum_bar);
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == PC_PRODUCERS / 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
    if (tid == 0 && s_abort) atomicOr(a.flags, 8);
}

// ---- pass 1 on the 5th-generation tensor cores ---------------------------------------------------------------------------
// D[row = token * 8 + head][key] per 64-key chunk: A = the rotated-query byte planes (128 rows x HD, written once), B = the
// key byte planes of the chunk (64 keys x HD, two stages), both K-major along the head dimension in the canonical layout.
// Sixteen warps produce the key planes and read the accumulators out (scores to the scratch, row maxima); one thread issues
// the MMAs, HD / 32 K steps x the byte pairs (16, or 9 where the queries and the chunk's keys fit 24 bits), first product of
// every accumulator of a chunk without accumulation.  The accumulators are single-buffered: the issuer waits until the
// previous chunk has been read out, the producers are already a chunk ahead.  grid (walks, Hkv, tiles).
constexpr int SC_WALK = 8, SC_STAGES = 2;
constexpr int SC_SLD = PT_CH + 2;           // row stride (int64) of the staged scores: 16-byte rows, lanes spread over the banks

// every producer thread learns whether all of them got through their waits (a named barrier with an AND reduction): the
// warps leave the chunk loop together, so none is left waiting at the plain barriers of the write-out
__device__ __forceinline__ bool pc_all_ok(bool ok) {
    uint32_t r;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 q, %1, 0;\n barrier.cta.red.and.pred p, 1, %2, q;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(r) : "r"((uint32_t)ok), "r"(PC_PRODUCERS) : "memory");
    return r != 0;
}

template <int HD>
__global__ void __launch_bounds__(PC_THREADS, 1) attn_tile_scores_tc_kernel(const AttnArgs a) {
    constexpr int HALF = HD / 2, Q_PLANE = PT_COLS * HD, K_PLANE = PT_CH * HD, K_STAGE = 4 * K_PLANE;
    extern __shared__ __align__(1024) unsigned char pc_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(pc_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[SC_STAGES], empty_bar[SC_STAGES], acc_bar, free_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_wide, s_qwide24, s_kwide24[SC_STAGES], s_mode[2];
    __shared__ long long s_max[PT_COLS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rep = a.H / a.Hkv, kv = blockIdx.y;
    const Tile T = pt_tile(a, (long long)gridDim.z - 1 - blockIdx.z);
    const long long c_first = T.lo_t / PT_CH + (long long)blockIdx.x * SC_WALK;
    if (c_first * PT_CH > T.pos_last) return;
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    const int n_chunks = (int)min((long long)SC_WALK, T.pos_last / PT_CH - c_first + 1);
    unsigned char *qd = smem;                                      // query byte planes [4][HD / 16][16 row groups][8 x 16 B]
    unsigned char *kd = qd + 4 * Q_PLANE;                          // key byte planes [2 stages][4][HD / 16][8 key groups][8 x 16 B]
    long long *sbuf = reinterpret_cast<long long *>(kd + SC_STAGES * K_STAGE);      // a chunk's scores [128 rows][SC_SLD] on their way out
    if (tid == 0) {
        s_abort = 0; s_wide = 0; s_qwide24 = 0;
        for (int s = 0; s < SC_STAGES; s++) {
            s_kwide24[s] = 0;
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&full_bar[s])), "r"(PC_PRODUCERS / 32));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&empty_bar[s])), "r"(1));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&acc_bar)), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pc_u32(&free_bar)), "r"(PC_PRODUCERS / 32));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < PT_COLS) s_max[tid] = INT64_MIN;
    if (warp == PC_PRODUCERS / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pc_u32(&s_tmem)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // rotated queries as byte planes in the canonical layout (row = token * 8 + head)
    {
        bool wide = false, wide24 = false;
        for (int idx0 = tid; idx0 < PT_COLS * HALF; idx0 += 4 * PC_THREADS) {      // four pairs per step: their loads are in flight together
            int64_t x0[4], x1[4], cs[4], sn[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int idx = idx0 + u * PC_THREADS, row = idx / HALF, i = idx - row * HALF, qi = row >> 3, h = row & 7;
                const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + HALF : 2 * i + 1;
                x0[u] = x1[u] = 0; cs[u] = sn[u] = 0;
                if (idx < PT_COLS * HALF && qi < T.nq && h < rep) {
                    const int64_t *src = a.q + ((T.t0 + qi) * a.H + kv * rep + h) * HD;
                    x0[u] = src[i0]; x1[u] = src[i1];
                    if (a.rope) { cs[u] = a.cos[(T.pos0 + qi) * HALF + i]; sn[u] = a.sin[(T.pos0 + qi) * HALF + i]; }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int idx = idx0 + u * PC_THREADS, row = idx / HALF, i = idx - row * HALF;
                if (idx >= PT_COLS * HALF) continue;
                const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + HALF : 2 * i + 1;
                int64_t y0 = x0[u], y1 = x1[u];
                if (a.rope) { y0 = (x0[u] * cs[u] - x1[u] * sn[u]) >> a.fa; y1 = (x0[u] * sn[u] + x1[u] * cs[u]) >> a.fa; }
                unsigned char *d0 = qd + (i0 >> 4) * (PT_COLS * 16) + (row >> 3) * 128 + (row & 7) * 16 + (i0 & 15);
                unsigned char *d1 = qd + (i1 >> 4) * (PT_COLS * 16) + (row >> 3) * 128 + (row & 7) * 16 + (i1 & 15);
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    d0[b * Q_PLANE] = (unsigned char)((uint32_t)(int32_t)y0 >> (8 * b));
                    d1[b * Q_PLANE] = (unsigned char)((uint32_t)(int32_t)y1 >> (8 * b));
                }
                wide |= y0 != (int32_t)y0 || y1 != (int32_t)y1;
                wide24 |= y0 < -(1 << 23) || y0 >= (1 << 23) || y1 < -(1 << 23) || y1 >= (1 << 23);
            }
        }
        if (wide) s_wide = 1;
        if (wide24) s_qwide24 = 1;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");         // the planes are read by the MMAs
    }
    __syncthreads();
    if (s_wide) {
        // a query value beyond int32: 64-bit wrapping products, one thread per (key, row); the rotated queries as int64 take
        // the place of every byte plane
        long long *q64 = reinterpret_cast<long long *>(smem);      // [128][HD]
        for (int idx = tid; idx < PT_COLS * HALF; idx += PC_THREADS) {
            const int row = idx / HALF, i = idx - row * HALF, qi = row >> 3, h = row & 7;
            const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + HALF : 2 * i + 1;
            int64_t x0 = 0, x1 = 0;
            if (qi < T.nq && h < rep) {
                const int64_t *src = a.q + ((T.t0 + qi) * a.H + kv * rep + h) * HD;
                x0 = src[i0]; x1 = src[i1];
                pt_rotate(a, T.pos0 + qi, i, x0, x1);
            }
            q64[row * HD + i0] = x0; q64[row * HD + i1] = x1;
        }
        __syncthreads();
        for (int w = 0; w < n_chunks; w++) {
            const long long l0 = (c_first + w) * PT_CH;
            for (int idx = tid; idx < PT_CH * PT_COLS; idx += PC_THREADS) {
                const int key = idx >> 7, row = idx & 127, qi = row >> 3, h = row & 7;
                const long long l = l0 + key, pos_q = T.pos0 + qi;
                if (qi >= T.nq || h >= rep || l > pos_q || l < pt_lo(a, pos_q)) continue;
                const int32_t *kk = a.kcache + ((long long)kv * a.Lmax + l) * HD;
                long long dot = 0;
                for (int j = 0; j < HD; j++) dot += q64[row * HD + j] * (long long)kk[j];
                const long long sc = ((dot >> a.fa) * a.inv_sqrt) >> a.fa;
                a.scores[((T.t0 + qi) * a.H + kv * rep + h) * Ls + l] = sc;
                atomicMax(&s_max[row], sc);
            }
        }
    } else if (warp < PC_PRODUCERS / 32) {
        const int r8 = lane >> 2, w4 = lane & 3;
        const int row = (warp & 3) * 32 + lane, qi = row >> 3, h = row & 7, cg = warp >> 2;      // read-out: TMEM lane and 16-key column group
        const long long pos_q = T.pos0 + qi, lo_q = pt_lo(a, pos_q);
        const bool row_ok = qi < T.nq && h < rep;
        const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        long long mloc = INT64_MIN;
        auto produce = [&](int ci) {                               // key planes of chunk ci into its stage
            const int s = ci % SC_STAGES;
            if (ci >= SC_STAGES && !pc_wait(&empty_bar[s], ((ci / SC_STAGES) - 1) & 1, &s_abort)) return false;
            unsigned char *stage = kd + (size_t)s * K_STAGE;
            const long long l0 = (c_first + ci) * PT_CH;
            bool fits = true;
#pragma unroll
            for (int u = 0; u < HD / 32; u++) {                    // (HD / 16) x 8 core matrices per plane, HD / 32 per warp
                const int cm = warp + 16 * u, kg = cm & 7, k16 = cm >> 3;
                const long long l = l0 + kg * 8 + r8;
                int4 v = make_int4(0, 0, 0, 0);
                if (l <= T.pos_last) v = __ldg(reinterpret_cast<const int4 *>(a.kcache + ((long long)kv * a.Lmax + l) * HD + k16 * 16) + w4);
                fits &= v.x >= -(1 << 23) && v.x < (1 << 23) && v.y >= -(1 << 23) && v.y < (1 << 23) &&
                        v.z >= -(1 << 23) && v.z < (1 << 23) && v.w >= -(1 << 23) && v.w < (1 << 23);
                uint32_t d[4];
                pt_planes((uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w, d[0], d[1], d[2], d[3]);
                unsigned char *dst = stage + k16 * (PT_CH * 16) + kg * 128 + r8 * 16 + w4 * 4;
#pragma unroll
                for (int b = 0; b < 4; b++) *reinterpret_cast<uint32_t *>(dst + b * K_PLANE) = d[b];
            }
            if (!__all_sync(0xffffffffu, fits) && lane == 0) atomicOr(&s_kwide24[s], 1);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pc_u32(&full_bar[s])) : "memory");
            return true;
        };
        bool ok = produce(0);
        for (int ci = 0; ci < n_chunks; ci++) {
            if (ok && ci + 1 < n_chunks) ok = produce(ci + 1);
            ok = ok && pc_wait(&acc_bar, ci & 1, &s_abort);
            if (!pc_all_ok(ok)) break;                             // uniform over the sixteen warps
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int ns = s_mode[ci & 1];                         // accumulators in use: 5 or 7
            const long long lc = (c_first + ci) * PT_CH, l0 = lc + cg * 16;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                int r[7][8];
#pragma unroll
                for (int s = 0; s < 7; s++)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[s][0]), "=r"(r[s][1]), "=r"(r[s][2]), "=r"(r[s][3]), "=r"(r[s][4]), "=r"(r[s][5]), "=r"(r[s][6]), "=r"(r[s][7])
                                 : "r"(tlane + s * PT_CH + cg * 16 + half * 8));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                long long sv[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    long long dot = 0;
                    if (ns == 7) dot = ((long long)r[6][j] * 256 + (long long)r[5][j]) * 256;
#pragma unroll
                    for (int s = 4; s >= 0; s--) dot = (s == 4 ? dot + (long long)r[4][j] : dot * 256 + (long long)r[s][j]);
                    const long long l = l0 + half * 8 + j;
                    sv[j] = ((dot >> a.fa) * a.inv_sqrt) >> a.fa;
                    if (row_ok && l <= pos_q && l >= lo_q) mloc = max(mloc, sv[j]);
                }
                longlong2 *dst = reinterpret_cast<longlong2 *>(sbuf + row * SC_SLD + cg * 16 + half * 8);
#pragma unroll
                for (int j = 0; j < 4; j++) dst[j] = make_longlong2(sv[2 * j], sv[2 * j + 1]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pc_u32(&free_bar)) : "memory");
            // the chunk's scores leave through shared memory so that a warp writes whole 512-byte rows (entries of keys a token
            // does not see are written too: they lie inside its row of the scratch and are never read)
            asm volatile("bar.sync 1, %0;" ::"r"(PC_PRODUCERS) : "memory");
            for (int rr = warp; rr < PT_COLS; rr += PC_PRODUCERS / 32) {
                const int q2 = rr >> 3, h2 = rr & 7;
                if (q2 < T.nq && h2 < rep)
                    *reinterpret_cast<longlong2 *>(a.scores + ((T.t0 + q2) * a.H + kv * rep + h2) * Ls + lc + 2 * lane) =
                        *reinterpret_cast<const longlong2 *>(sbuf + rr * SC_SLD + 2 * lane);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(PC_PRODUCERS) : "memory");
        }
        if (mloc != INT64_MIN) atomicMax(&s_max[row], mloc);
    } else {
        // ================= MMA issuer ===========================================================================================
        if (lane == 0) {
            constexpr uint32_t IDESC = (2u << 4) | ((uint32_t)(PT_CH >> 3) << 17) | ((uint32_t)(PT_COLS >> 4) << 24);      // + (1 << 7) A signed, (1 << 10) B signed
            const bool q_narrow = s_qwide24 == 0;
            bool ok = true;
            for (int ci = 0; ci < n_chunks && ok; ci++) {
                const int s = ci % SC_STAGES;
                ok = pc_wait(&full_bar[s], (ci / SC_STAGES) & 1, &s_abort);
                if (ok && ci > 0) ok = pc_wait(&free_bar, (ci - 1) & 1, &s_abort);      // the previous chunk's scores have left TMEM
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const bool narrow = q_narrow && s_kwide24[s] == 0;
                s_kwide24[s] = 0;                                  // for the next chunk of this stage (ordered by the commit below)
                s_mode[ci & 1] = narrow ? 5 : 7;
                const uint32_t stage = pc_u32(kd + (size_t)s * K_STAGE);
                const uint64_t dq0 = pc_desc(pc_u32(qd), PT_COLS * 16, 128), dk0 = pc_desc(stage, PT_CH * 16, 128);
                auto issue = [&](auto nb_c) {
                    constexpr int NB = decltype(nb_c)::value;
#pragma unroll
                    for (int ks = 0; ks < HD / 32; ks++)
#pragma unroll
                        for (int b = 0; b < NB; b++)
#pragma unroll
                            for (int aa = 0; aa < NB; aa++) {
                                const bool first = ks == 0 && (b == 0 || aa == NB - 1);       // first product into accumulator aa + b
                                const uint64_t dq = dq0 + (uint64_t)((aa * Q_PLANE + ks * 2 * PT_COLS * 16) >> 4);
                                const uint64_t dk = dk0 + (uint64_t)((b * K_PLANE + ks * 2 * PT_CH * 16) >> 4);
                                pc_mma(tmem + (aa + b) * PT_CH, dq, dk, IDESC | (aa == NB - 1 ? 1u << 7 : 0u) | (b == NB - 1 ? 1u << 10 : 0u), first ? 0u : 1u);
                            }
                };
                if (narrow) issue(std::integral_constant<int, 3>{}); else issue(std::integral_constant<int, 4>{});
                pc_commit(&empty_bar[s]);
                pc_commit(&acc_bar);
            }
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == PC_PRODUCERS / 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
    if (tid < PT_COLS && s_max[tid] != INT64_MIN) {
        const int qi = tid >> 3, h = tid & 7;
        atomicMax(a.hmax + (T.t0 + qi) * a.H + kv * rep + h, s_max[tid]);
    }
    if (tid == 0 && s_abort) atomicOr(a.flags, 8);
}

template <int HD>
cudaError_t scores_launch(const AttnArgs &a, unsigned walks, unsigned tiles, cudaStream_t s) {
    constexpr size_t smem = (size_t)4 * PT_COLS * (HD + 16) + (size_t)2 * 4 * PT_CH * (HD + 16);
    static_assert(smem >= (size_t)PT_COLS * HD * 8, "the int64 queries of the scalar path overlay the byte planes");
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tile_scores_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    attn_tile_scores_kernel<HD><<<dim3(walks, a.Hkv, tiles), PT_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

template <int HD>
cudaError_t pv_launch(const AttnArgs &a, unsigned tiles, cudaStream_t s) {
    constexpr size_t smem = (size_t)4 * HD * PT_PLD + (size_t)3 * PT_COLS * PT_PLD + (size_t)PT_CH * HD * 4;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tile_pv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    attn_tile_pv_kernel<HD><<<dim3(1, a.Hkv, tiles), PT_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

template <int HD>
cudaError_t scores_tc_launch(const AttnArgs &a, unsigned walks, unsigned tiles, cudaStream_t s) {
    constexpr size_t smem = (size_t)4 * PT_COLS * HD + (size_t)SC_STAGES * 4 * PT_CH * HD + (size_t)PT_COLS * SC_SLD * 8 + 1024;
    static_assert(smem - 1024 >= (size_t)PT_COLS * HD * 8, "the int64 queries of the scalar path overlay the byte planes");
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tile_scores_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    attn_tile_scores_tc_kernel<HD><<<dim3(walks, a.Hkv, tiles), PC_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

template <int HD>
cudaError_t pv_tc_launch(const AttnArgs &a, unsigned tiles, cudaStream_t s) {
    constexpr size_t smem = (size_t)PC_STAGES * PC_STAGE + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tile_pv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    attn_tile_pv_tc_kernel<HD><<<dim3(HD / PC_N, a.Hkv, tiles), PC_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

}  // namespace

int g_attn_tile_tc = 1;                    // 1: probability x value of a prefill on tcgen05 where the key span allows, 0: mma.sync tiles

bool attn_tiles_ok(const AttnArgs &a) {
    const int rep = a.Hkv > 0 ? a.H / a.Hkv : 0;
    return a.batch >= 4 && a.seq_stride == 0 && rep >= 1 && rep <= PT_HEADS && (a.hd == 64 || a.hd == 128) && a.fa <= 23 && !a.pos_dev;
}

cudaError_t launch_attn_tile_scores(const AttnArgs &a, cudaStream_t s) {
    if (!attn_tiles_ok(a)) return cudaErrorInvalidValue;
    const unsigned tiles = (unsigned)((a.batch + PT_Q - 1) / PT_Q);
    long long span = a.pos + a.batch;                              // keys the last token sees, plus the tile's own tokens under a window
    if (a.window > 0 && span > a.window + PT_Q) span = a.window + PT_Q;
    const int walk = g_attn_tile_tc != 0 ? SC_WALK : PT_WALK;
    const unsigned walks = (unsigned)((span / PT_CH + 2 + walk - 1) / walk);
    const cudaError_t e = g_attn_tile_tc != 0 ? (a.hd == 128 ? scores_tc_launch<128>(a, walks, tiles, s) : scores_tc_launch<64>(a, walks, tiles, s))
                                              : (a.hd == 128 ? scores_launch<128>(a, walks, tiles, s) : scores_launch<64>(a, walks, tiles, s));
    note_launch();
    return e;
}

cudaError_t launch_attn_tile_exp(const AttnArgs &a, cudaStream_t s) {
    if (!attn_tiles_ok(a)) return cudaErrorInvalidValue;
    const long long rows = (long long)a.batch * a.H;
    attn_tile_exp_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(a);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_attn_tile_pv(const AttnArgs &a, cudaStream_t s) {
    if (!attn_tiles_ok(a) || !a.out) return cudaErrorInvalidValue;
    const unsigned tiles = (unsigned)((a.batch + PT_Q - 1) / PT_Q);
    long long span = a.pos + a.batch;                              // keys a tile can walk
    if (a.window > 0 && span > a.window + PT_Q) span = a.window + PT_Q;
    const bool tc = g_attn_tile_tc != 0 && span / PT_CH + 2 <= PC_MAX_CHUNKS;      // the int32 accumulators run over the whole span
    const cudaError_t e = tc ? (a.hd == 128 ? pv_tc_launch<128>(a, tiles, s) : pv_tc_launch<64>(a, tiles, s))
                             : (a.hd == 128 ? pv_launch<128>(a, tiles, s) : pv_launch<64>(a, tiles, s));
    note_launch();
    return e;
}

}  // namespace iie
