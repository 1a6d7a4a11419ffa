// Integer attention for one new token over a KV cache, plus the two small ends of a decode step
// (embedding row, arg-max of the logits).
//
// Arithmetic of north-mini-code/src/nmc/cohere2.py:324-354 (attention_cached) with
// _bonsai/fixedpoint.py:99-133 (fixed_point_softmax) and _bonsai/rope.py:79-100 / rope_v2.py:92-117:
//     score_l = (((q . k_l) >> fa) * inv_sqrt) >> fa          over the visible keys lo..pos
//     e_l     = 2^-(((min(max - score_l, clip)) * log2e) >> fa)          (cubic fixed-point 2^-f)
//     p_l     = (e_l << fa) // sum(e)
//     out_d   = (sum_l p_l v_{l,d}) >> fa
// Masked keys carry the sentinel -(2^(fa+30)) in the reference; their e is exactly 0 and the row maximum is
// always a visible key, so skipping them gives the same bytes.
//
// The floors make the softmax non-linear, so the three passes need the row maximum and the normaliser of ALL
// visible keys: scores + max, exponentials + sum, probabilities x values are three launches over
// (KV head, key chunk) CTAs; a CTA serves every query head of its KV head so K and V are read once.
// The first pass also rotates the query heads (into shared memory, the caller's q is not modified) and, in the
// CTA that owns the new position, rotates the new key and appends key and value to the cache; the last CTA of
// the third pass writes the result (optionally as digit planes for the following product) and resets the
// shared statistics, so a call is exactly three launches.
// The cache holds K (after rotation) and V as int32: values outside int32 raise flag bit 2 (the reference bank
// stores them the same way and refuses such values).
#include <cooperative_groups.h>

#include <algorithm>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"
#include "norm.cuh"

namespace cg = cooperative_groups;

namespace iie {

int g_attn_fused = 1;                      // 1: one cooperative launch where every CTA fits on the device (one CTA per SM where the chunks fit
                                           // shared memory), 2: the same without the one-CTA-per-SM form, 0: always three launches

namespace {

constexpr int AT_CH = 64;                   // keys per CTA
constexpr int AT_MAXREP = 16;               // query heads per KV head

// position of the new token and first visible key: from the device cell when the caller replays a captured graph
// Returns false (uniformly over the grid) when the device cell holds a position beyond the host bound the grids were
// sized for, or beyond the cache rows: the kernel then raises flag bit 4 and returns without touching the cache.
__device__ __forceinline__ bool at_span(const AttnArgs &a, long long &pos, long long &lo) {
    pos = a.pos_dev ? (long long)*a.pos_dev : a.pos;
    lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    return !(a.pos_dev && (pos < 0 || pos > a.pos || pos >= a.Lmax));
}
__device__ __forceinline__ void at_refuse(const AttnArgs &a) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) atomicOr(a.flags, 16);
}

// several new tokens in one launch: blockIdx.z is the token; shift every per-token pointer to it.  Prefill (seq_stride == 0):
// the tokens are consecutive positions of ONE sequence and share its cache.  Batched decode (seq_stride > 0): token i is
// the new token of sequence i, all at position pos, each sequence with its own cache seq_stride elements further on.
__device__ __forceinline__ void at_batch(AttnArgs &a) {
    if (a.batch <= 0) return;
    const long long i = blockIdx.z, Ls = a.Ls ? a.Ls : a.Lmax;
    if (a.seq_stride > 0) { a.kcache += i * a.seq_stride; a.vcache += i * a.seq_stride; }
    else a.pos += i;
    a.lo = (a.window > 0 && a.pos - a.window + 1 > 0) ? a.pos - a.window + 1 : 0;
    a.q += i * a.H * a.hd;
    a.scores += i * a.H * Ls; a.e += i * a.H * Ls; a.hmax += i * a.H; a.Z += i * a.H;
    if (a.out) a.out += i * a.H * a.hd;
}

// rotation of one (x0, x1) pair with the table row of `pos`
__device__ __forceinline__ void at_rotate(const AttnArgs &a, long long pos, int i, int64_t &x0, int64_t &x1) {
    if (!a.rope) return;
    const int half = a.hd / 2;
    const int64_t c = a.cos[pos * half + i], s = a.sin[pos * half + i];
    const int64_t y0 = (x0 * c - x1 * s) >> a.fa, y1 = (x0 * s + x1 * c) >> a.fa;
    x0 = y0; x1 = y1;
}

// Copy n 16-byte vectors from global to shared memory with eight loads of a thread in flight before the first
// store (a plain loop would wait for every load in turn).  dst_of(i) gives the destination vector index.
template <typename F>
__device__ __forceinline__ void at_stage(const int4 *src, int n, int tid, int nth, int32_t *dst_base, F dst_of) {
    for (int i0 = 0; i0 < n; i0 += nth * 8) {
        int4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) { const int i = i0 + u * nth + tid; if (i < n) v[u] = src[i]; }
#pragma unroll
        for (int u = 0; u < 8; u++) { const int i = i0 + u * nth + tid; if (i < n) *reinterpret_cast<int4 *>(dst_base + dst_of(i)) = v[u]; }
    }
}

__global__ void attn_reset_kernel(long long *hmax, unsigned long long *Z, long long *acc, unsigned *ticket, int H, int hd) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) { hmax[i] = INT64_MIN; Z[i] = 0ULL; }
    for (int i = threadIdx.x; i < H * hd; i += blockDim.x) acc[i] = 0;
    for (int i = threadIdx.x; i < 257; i += blockDim.x) ticket[i] = 0u;        // the ticket and the per-KV-head barrier counters
}

// pass 1: scores of AT_CH keys for the `rep` query heads of one KV head; the keys are staged in shared memory and
// each thread owns one key for a quarter of the query heads.  Every CTA rotates
// its query heads into shared memory; the CTA whose chunk holds `pos` rotates the new key and appends key and
// value to the cache first.
__global__ void __launch_bounds__(256) attn_scores_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }
    at_batch(a);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    extern __shared__ __align__(16) long long at_q[];     // [rep][hd] int64, then [rep][hd] int32, then the key chunk
    __shared__ long long s_max[AT_MAXREP];
    __shared__ int s_wide;
    const int kv = blockIdx.y, rep = a.H / a.Hkv, tid = threadIdx.x, lane = tid & 31;
    const int half = a.hd / 2;
    const long long l0 = a.lo + (long long)blockIdx.x * AT_CH, l1 = min(l0 + AT_CH, a.pos + 1);
    if (a.batch && l0 > a.pos) return;                     // prefill: a chunk past this token's position
    int32_t *q32 = reinterpret_cast<int32_t *>(at_q + rep * a.hd);
    int32_t *sk = q32 + rep * a.hd;
    if (tid == 0) s_wide = 0;
    if (tid < AT_MAXREP) s_max[tid] = INT64_MIN;
    __syncthreads();
    bool wide = false;
    for (int idx = tid; idx < rep * half; idx += blockDim.x) {
        const int r = idx / half, i = idx - r * half;
        const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
        const int64_t *src = a.q + (long long)(kv * rep + r) * a.hd;
        int64_t x0 = src[i0], x1 = src[i1];
        at_rotate(a, a.pos, i, x0, x1);
        at_q[r * a.hd + i0] = x0; at_q[r * a.hd + i1] = x1;
        q32[r * a.hd + i0] = (int32_t)x0; q32[r * a.hd + i1] = (int32_t)x1;
        wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
    }
    if (wide) s_wide = 1;
    if (!a.batch && l0 <= a.pos && a.pos < l0 + AT_CH) {  // this CTA owns the new token's cache row
        bool bad = false;
        for (int i = tid; i < half; i += blockDim.x) {
            const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
            int64_t x0 = a.k[kv * a.hd + i0], x1 = a.k[kv * a.hd + i1];
            at_rotate(a, a.pos, i, x0, x1);
            bad |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
            int32_t *dst = a.kcache + ((long long)kv * a.Lmax + a.pos) * a.hd;
            dst[i0] = (int32_t)x0; dst[i1] = (int32_t)x1;
        }
        for (int i = tid; i < a.hd; i += blockDim.x) {
            const int64_t v = a.v[kv * a.hd + i];
            bad |= v != (int32_t)v;
            a.vcache[((long long)kv * a.Lmax + a.pos) * a.hd + i] = (int32_t)v;
        }
        if (bad) atomicOr(a.flags, 4);
    }
    __syncthreads();                                       // q in shared memory; the new row is in the cache
    // stage the chunk's keys: coalesced 16-byte loads; rows padded by four words keep them 16-byte aligned and put
    // the eight rows of a quarter-warp's vector load on different banks
    const int nk = (int)max(0LL, l1 - l0), ld = a.hd + 4, vec_per_row = a.hd / 4;
    at_stage(reinterpret_cast<const int4 *>(a.kcache + ((long long)kv * a.Lmax + l0) * a.hd), nk * vec_per_row, tid, blockDim.x, sk,
             [&](int i) { const int row = i / vec_per_row; return row * ld + (i - row * vec_per_row) * 4; });
    __syncthreads();
    // thread -> (key, head group): 64 keys x 4 groups; a group takes `hpt` consecutive query heads
    const int key = tid & (AT_CH - 1), hg = tid / AT_CH, n_hg = blockDim.x / AT_CH, hpt = (rep + n_hg - 1) / n_hg;
    const bool use_wide = s_wide != 0;
    for (int r0 = hg * hpt; r0 < min(rep, (hg + 1) * hpt); r0 += 2) {
        const bool two = r0 + 1 < min(rep, (hg + 1) * hpt);
        long long d0 = 0, d1 = 0;
        if (key < nk) {
            const int32_t *kk = sk + key * ld;
            if (!use_wide) {                               // every query value fits 32 bits: one wide multiply-add per term
                const int32_t *qa = q32 + r0 * a.hd, *qb = q32 + (two ? r0 + 1 : r0) * a.hd;
                for (int j = 0; j < a.hd; j += 4) {
                    const int4 k4 = *reinterpret_cast<const int4 *>(kk + j);
                    const int4 a4 = *reinterpret_cast<const int4 *>(qa + j), b4 = *reinterpret_cast<const int4 *>(qb + j);
                    d0 += (long long)a4.x * k4.x; d0 += (long long)a4.y * k4.y; d0 += (long long)a4.z * k4.z; d0 += (long long)a4.w * k4.w;
                    d1 += (long long)b4.x * k4.x; d1 += (long long)b4.y * k4.y; d1 += (long long)b4.z * k4.z; d1 += (long long)b4.w * k4.w;
                }
            } else {
                const long long *qa = at_q + r0 * a.hd, *qb = at_q + (two ? r0 + 1 : r0) * a.hd;
                for (int j = 0; j < a.hd; j++) { const long long kj = kk[j]; d0 += qa[j] * kj; d1 += qb[j] * kj; }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            if (u == 1 && !two) break;
            const int r = r0 + u;
            long long sc = INT64_MIN;
            if (key < nk) {
                sc = (((u ? d1 : d0) >> a.fa) * a.inv_sqrt) >> a.fa;
                a.scores[(long long)(kv * rep + r) * Ls + l0 + key] = sc;
            }
            long long m = sc;
#pragma unroll
            for (int s2 = 16; s2 > 0; s2 >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s2));
            if (lane == 0 && m != INT64_MIN) atomicMax(&s_max[r], m);
        }
    }
    __syncthreads();
    if (tid < rep && s_max[tid] != INT64_MIN) atomicMax(a.hmax + kv * rep + tid, s_max[tid]);
}

// pass 2: exponentials and their sum
__global__ void __launch_bounds__(256) attn_exp_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }
    at_batch(a);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    __shared__ unsigned long long s_sum[8];
    const int h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long l = a.lo + (long long)blockIdx.x * 256 + tid;
    unsigned long long e = 0;
    if (l <= a.pos) {
        const long long m = a.hmax[h], s = a.scores[(long long)h * Ls + l];
        long long dlt = m - s;
        dlt = dlt < a.clip ? dlt : a.clip;
        e = (unsigned long long)exp2_neg_fixed((dlt * a.log2e) >> a.fa, a.fa);
        a.e[(long long)h * Ls + l] = (int32_t)e;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) e += __shfl_xor_sync(0xffffffffu, e, s);
    if (lane == 0) s_sum[warp] = e;
    __syncthreads();
    if (tid == 0) {
        unsigned long long t = 0;
        for (int i = 0; i < 8; i++) t += s_sum[i];
        if (t) atomicAdd(a.Z + h, t);
    }
}

// pass 3: probabilities x values, partial sums added into acc.  The CTA that finishes last shifts, writes the
// result (and, on request, its digit planes) and returns the shared statistics to their initial state.
__global__ void __launch_bounds__(256) attn_pv_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    extern __shared__ __align__(16) int32_t at_v[];        // [AT_CH][hd] values, then [AT_CH][AT_MAXREP] probabilities
    __shared__ int s_last, s_nl;
    const int kv = blockIdx.y, rep = a.H / a.Hkv, tid = threadIdx.x;
    const long long l0 = a.lo + (long long)blockIdx.x * AT_CH, l1 = min(l0 + AT_CH, a.pos + 1);
    const int nk = (int)max(0LL, l1 - l0);
    int32_t *s_p = at_v + AT_CH * a.hd;                    // p <= 2^fa fits 32 bits
    for (int i = tid; i < AT_MAXREP * AT_CH; i += blockDim.x) {
        const int j = i / AT_MAXREP, r = i - j * AT_MAXREP;
        int32_t p = 0;
        if (j < nk && r < rep) {
            const int h = kv * rep + r;
            const unsigned long long z = a.Z[h];
            const unsigned long long e = (unsigned long long)(unsigned)a.e[(long long)h * Ls + l0 + j];
            p = z ? (int32_t)((e << a.fa) / z) : 0;
        }
        s_p[i] = p;
    }
    at_stage(reinterpret_cast<const int4 *>(a.vcache + ((long long)kv * a.Lmax + l0) * a.hd), nk * (a.hd / 4), tid, blockDim.x, at_v,
             [](int i) { return i * 4; });
    if (tid == 0) s_nl = 1;
    __syncthreads();
    // thread -> (column d, head group): a group owns four consecutive query heads per pass
    const int G = blockDim.x / a.hd, grp = tid / a.hd, d = tid - grp * a.hd;
    if (grp < G && nk > 0) {
        for (int r0 = grp * 4; r0 < rep; r0 += G * 4) {
            long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
            for (int j = 0; j < nk; j++) {
                const int32_t v = at_v[j * a.hd + d];
                const int4 p4 = *reinterpret_cast<const int4 *>(s_p + j * AT_MAXREP + r0);
                c0 += (long long)p4.x * v; c1 += (long long)p4.y * v; c2 += (long long)p4.z * v; c3 += (long long)p4.w * v;
            }
            const long long cs[4] = {c0, c1, c2, c3};
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u < rep && cs[u] != 0)
                    atomicAdd(reinterpret_cast<unsigned long long *>(a.acc + (long long)(kv * rep + r0 + u) * a.hd + d), (unsigned long long)cs[u]);
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.ticket, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const long long n = (long long)a.H * a.hd;
    int nl = 1;
    bool over = false;
    for (long long i0 = 0; i0 < n; i0 += (long long)blockDim.x * 8) {
        long long yv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {                     // all eight loads in flight before any is used
            const long long i = i0 + (long long)u * blockDim.x + tid;
            yv[u] = i < n ? __ldcg(a.acc + i) : 0;
        }
#pragma unroll 1
        for (int u = 0; u < 8; u++) {
            const long long i = i0 + (long long)u * blockDim.x + tid;
            if (i >= n) continue;
            const long long y = yv[u] >> a.fa;
            if (a.out) a.out[i] = y;
            if (a.out_limbs) {
                bool ok;
                const uint64_t dg = balanced_digits8(y, ok);
                over |= !ok;
                nl = max(nl, digits_used(dg));
#pragma unroll
                for (int l = 0; l < 8; l++) a.out_limbs[l * n + i] = (int8_t)(dg >> (8 * l));
            }
            a.acc[i] = 0;
        }
    }
    if (over) atomicOr(a.flags, 1);
    if (a.out_limbs) atomicMax(&s_nl, nl);
    for (int i = tid; i < a.H; i += blockDim.x) { a.hmax[i] = INT64_MIN; a.Z[i] = 0ULL; }
    __syncthreads();
    if (tid == 0) { *a.ticket = 0u; if (a.out_nl) *a.out_nl = s_nl; }
}

// several tokens, before the passes: rotate the new keys and append keys and values of all `batch` tokens (to one cache at
// consecutive positions, or each to its own sequence's cache at position pos); grid (batch, Hkv)
__global__ void __launch_bounds__(128) attn_append_kernel(const AttnArgs a) {
    const long long i = blockIdx.x, pos = a.seq_stride > 0 ? a.pos : a.pos + i, seq = a.seq_stride > 0 ? i * a.seq_stride : 0;
    const int kv = blockIdx.y, tid = threadIdx.x, half = a.hd / 2;
    const int64_t *ks = a.k + (i * a.Hkv + kv) * a.hd, *vs = a.v + (i * a.Hkv + kv) * a.hd;
    int32_t *kd = a.kcache + seq + ((long long)kv * a.Lmax + pos) * a.hd, *vd = a.vcache + seq + ((long long)kv * a.Lmax + pos) * a.hd;
    bool bad = false;
    for (int j = tid; j < half; j += blockDim.x) {
        const int i0 = a.rope == 2 ? j : 2 * j, i1 = a.rope == 2 ? j + half : 2 * j + 1;
        int64_t x0 = ks[i0], x1 = ks[i1];
        at_rotate(a, pos, j, x0, x1);
        bad |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
        kd[i0] = (int32_t)x0; kd[i1] = (int32_t)x1;
    }
    for (int j = tid; j < a.hd; j += blockDim.x) {
        const int64_t v = vs[j];
        bad |= v != (int32_t)v;
        vd[j] = (int32_t)v;
    }
    if (bad) atomicOr(a.flags, 4);
    const int rep = a.H / a.Hkv;                           // statistics of this token's query heads on this KV head
    for (int r = tid; r < rep; r += blockDim.x) { a.hmax[i * a.H + kv * rep + r] = INT64_MIN; a.Z[i * a.H + kv * rep + r] = 0ULL; }
}

// prefill / batched pass 3: one CTA per (token, KV head[, share of the chunks]) walks key chunks; the next chunk's values
// stream in (cp.async, second buffer) while the current one is multiplied.  A thread owns two output dimensions of four
// query heads for one part of a chunk's keys (one value load and one probability load per eight multiply-adds); the
// parts are added through shared memory at the end.  grid (pv_splits or 1, Hkv, batch)
__global__ void __launch_bounds__(256) attn_pv_rows_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    at_batch(a);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    extern __shared__ __align__(16) int32_t at_v[];        // two value buffers [AT_CH][hd], probabilities [AT_CH][AT_MAXREP], sums
    const int kv = blockIdx.y, rep = a.H / a.Hkv, tid = threadIdx.x, hd = a.hd, half = hd / 2;
    int32_t *s_p = at_v + 2 * AT_CH * hd;
    long long *red = reinterpret_cast<long long *>(s_p + AT_CH * AT_MAXREP);            // [KQ][AT_MAXREP][hd]
    const int KQ = blockDim.x / hd;                        // parts of a chunk's keys
    const int dp = tid % half, hh = (tid / half) & 1, kq = tid / hd;
    // with pv_splits > 1 this CTA takes a contiguous share of the key chunks and leaves raw sums for attn_pv_finish_kernel
    const int splits = a.pv_splits > 1 ? a.pv_splits : 1;
    const long long n_chunks = (a.pos - a.lo) / AT_CH + 1, per = (n_chunks + splits - 1) / splits;
    const long long c_lo = (long long)blockIdx.x * per, c_hi = min(n_chunks, c_lo + per);
    const int vec_per_chunk = AT_CH * hd / 4;
    auto request = [&](long long c) {                      // values of chunk c into buffer c & 1
        const long long l0 = a.lo + c * AT_CH;
        const int nk = (int)min((long long)AT_CH, a.pos + 1 - l0);
        const int4 *src = reinterpret_cast<const int4 *>(a.vcache + ((long long)kv * a.Lmax + l0) * hd);
        int32_t *dst = at_v + (size_t)(c & 1) * AT_CH * hd;
        for (int i = tid; i < nk * (hd / 4) && i < vec_per_chunk; i += blockDim.x) {
            const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + i * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int rbase = 0; rbase < rep; rbase += 8) {                          // eight query heads per pass
        long long c[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};
        if (c_lo < c_hi) request(c_lo);
        for (long long ch = c_lo; ch < c_hi; ch++) {
            const long long l0 = a.lo + ch * AT_CH;
            const int nk = (int)min((long long)AT_CH, a.pos + 1 - l0);
            __syncthreads();                                                // the previous chunk's probabilities and its buffer are free
            if (ch + 1 < c_hi) request(ch + 1);
            for (int i = tid; i < 8 * AT_CH; i += blockDim.x) {
                const int j = i >> 3, r = rbase + (i & 7);
                int32_t p = 0;
                if (j < nk && r < rep) {
                    const int h = kv * rep + r;
                    const unsigned long long z = a.Z[h];
                    const unsigned long long e = (unsigned long long)(unsigned)a.e[(long long)h * Ls + l0 + j];
                    p = z ? (int32_t)((e << a.fa) / z) : 0;
                }
                s_p[i] = p;
            }
            if (ch + 1 < c_hi) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            const int32_t *sv = at_v + (size_t)(ch & 1) * AT_CH * hd;
            const int perk = (nk + KQ - 1) / KQ, j0 = min(nk, kq * perk), j1 = min(nk, j0 + perk);
            for (int j = j0; j < j1; j++) {
                const int2 v2 = *reinterpret_cast<const int2 *>(sv + (size_t)j * hd + 2 * dp);
                const int4 p4 = *reinterpret_cast<const int4 *>(s_p + j * 8 + 4 * hh);
                c[0][0] += (long long)p4.x * v2.x; c[0][1] += (long long)p4.x * v2.y;
                c[1][0] += (long long)p4.y * v2.x; c[1][1] += (long long)p4.y * v2.y;
                c[2][0] += (long long)p4.z * v2.x; c[2][1] += (long long)p4.z * v2.y;
                c[3][0] += (long long)p4.w * v2.x; c[3][1] += (long long)p4.w * v2.y;
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 4; u++)
            *reinterpret_cast<longlong2 *>(red + ((size_t)kq * 8 + 4 * hh + u) * hd + 2 * dp) = make_longlong2(c[u][0], c[u][1]);
        __syncthreads();
        for (int o = tid; o < 8 * hd; o += blockDim.x) {
            const int r = rbase + o / hd, d = o % hd;
            if (r >= rep) continue;
            long long sum = 0;
            for (int g = 0; g < KQ; g++) sum += red[(size_t)g * 8 * hd + o];
            const long long oo = (long long)(kv * rep + r) * hd + d;
            if (splits == 1) a.out[oo] = sum >> a.fa;
            else a.pv_part[(((long long)blockIdx.z * splits + blockIdx.x) * a.H) * hd + oo] = sum;
        }
    }
}

// out = (sum of the pv_splits partial sums) >> fa, one thread per output of every token
__global__ void attn_pv_finish_kernel(const AttnArgs a) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, per_tok = (long long)a.H * a.hd;
    if (i >= (long long)a.batch * per_tok) return;
    const long long tok = i / per_tok, o = i - tok * per_tok;
    long long sum = 0;
    for (int sidx = 0; sidx < a.pv_splits; sidx++) sum += a.pv_part[((tok * a.pv_splits + sidx) * a.H) * a.hd + o];
    a.out[i] = sum >> a.fa;
}

// The three passes in ONE cooperative launch (all CTAs co-resident, two grid-wide barriers): scores and
// exponentials stay in registers, the value chunk is requested into shared memory together with the key chunk so
// its latency is hidden behind the first two passes, and nothing but the statistics goes through global memory.
__global__ void __launch_bounds__(256) attn_fused_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }
    cg::grid_group grid = cg::this_grid();
    extern __shared__ __align__(16) long long at_q[];     // q int64 [rep][hd], q int32 [rep][hd], keys [CH][hd+4], values [CH][hd], p [CH][MAXREP]
    __shared__ long long s_max[AT_MAXREP];
    __shared__ unsigned long long s_z[AT_MAXREP];
    __shared__ int s_wide;
    const int kv = blockIdx.y, rep = a.H / a.Hkv, tid = threadIdx.x, lane = tid & 31;
    const int half = a.hd / 2;
    const long long l0 = a.lo + (long long)blockIdx.x * AT_CH, l1 = min(l0 + AT_CH, a.pos + 1);
    const int nk = (int)max(0LL, l1 - l0), ld = a.hd + 4, vec_per_row = a.hd / 4;
    int32_t *q32 = reinterpret_cast<int32_t *>(at_q + rep * a.hd);
    int32_t *sk = q32 + rep * a.hd;
    int32_t *sv = sk + AT_CH * ld;
    int32_t *s_p = sv + AT_CH * a.hd;
    if (tid == 0) s_wide = 0;
    if (tid < AT_MAXREP) { s_max[tid] = INT64_MIN; s_z[tid] = 0ULL; }
    __syncthreads();
    // programmatic dependent launch: everything above touched only shared memory and the position cell (written a
    // whole step earlier); q, k, v come from the product launched just before
    if (a.pdl) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }
    bool wide = false;
    for (int idx = tid; idx < rep * half; idx += blockDim.x) {
        const int r = idx / half, i = idx - r * half;
        const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
        const int64_t *src = a.q + (long long)(kv * rep + r) * a.hd;
        int64_t x0 = src[i0], x1 = src[i1];
        at_rotate(a, a.pos, i, x0, x1);
        at_q[r * a.hd + i0] = x0; at_q[r * a.hd + i1] = x1;
        q32[r * a.hd + i0] = (int32_t)x0; q32[r * a.hd + i1] = (int32_t)x1;
        wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
    }
    if (wide) s_wide = 1;
    if (!a.batch && l0 <= a.pos && a.pos < l0 + AT_CH) {  // this CTA owns the new token's cache row
        bool bad = false;
        for (int i = tid; i < half; i += blockDim.x) {
            const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
            int64_t x0 = a.k[kv * a.hd + i0], x1 = a.k[kv * a.hd + i1];
            at_rotate(a, a.pos, i, x0, x1);
            bad |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
            int32_t *dst = a.kcache + ((long long)kv * a.Lmax + a.pos) * a.hd;
            dst[i0] = (int32_t)x0; dst[i1] = (int32_t)x1;
        }
        for (int i = tid; i < a.hd; i += blockDim.x) {
            const int64_t v = a.v[kv * a.hd + i];
            bad |= v != (int32_t)v;
            a.vcache[((long long)kv * a.Lmax + a.pos) * a.hd + i] = (int32_t)v;
        }
        if (bad) atomicOr(a.flags, 4);
    }
    __syncthreads();
    at_stage(reinterpret_cast<const int4 *>(a.kcache + ((long long)kv * a.Lmax + l0) * a.hd), nk * vec_per_row, tid, blockDim.x, sk,
             [&](int i) { const int row = i / vec_per_row; return row * ld + (i - row * vec_per_row) * 4; });
    at_stage(reinterpret_cast<const int4 *>(a.vcache + ((long long)kv * a.Lmax + l0) * a.hd), nk * vec_per_row, tid, blockDim.x, sv,
             [](int i) { return i * 4; });
    __syncthreads();
    // ---- pass 1: thread -> (key, head group); a group takes `hpt` (<= 4) consecutive query heads -------------------
    const int key = tid & (AT_CH - 1), hg = tid / AT_CH, n_hg = blockDim.x / AT_CH, hpt = (rep + n_hg - 1) / n_hg;
    const int r_lo = hg * hpt, r_hi = min(rep, (hg + 1) * hpt);
    const bool use_wide = s_wide != 0;
    long long sc[4] = {INT64_MIN, INT64_MIN, INT64_MIN, INT64_MIN};
#pragma unroll
    for (int pr = 0; pr < 2; pr++) {
        const int r0 = r_lo + 2 * pr;
        if (r0 >= r_hi) break;
        const bool two = r0 + 1 < r_hi;
        long long d0 = 0, d1 = 0;
        if (key < nk) {
            const int32_t *kk = sk + key * ld;
            if (!use_wide) {
                const int32_t *qa = q32 + r0 * a.hd, *qb = q32 + (two ? r0 + 1 : r0) * a.hd;
                for (int j = 0; j < a.hd; j += 4) {
                    const int4 k4 = *reinterpret_cast<const int4 *>(kk + j);
                    const int4 a4 = *reinterpret_cast<const int4 *>(qa + j), b4 = *reinterpret_cast<const int4 *>(qb + j);
                    d0 += (long long)a4.x * k4.x; d0 += (long long)a4.y * k4.y; d0 += (long long)a4.z * k4.z; d0 += (long long)a4.w * k4.w;
                    d1 += (long long)b4.x * k4.x; d1 += (long long)b4.y * k4.y; d1 += (long long)b4.z * k4.z; d1 += (long long)b4.w * k4.w;
                }
            } else {
                const long long *qa = at_q + r0 * a.hd, *qb = at_q + (two ? r0 + 1 : r0) * a.hd;
                for (int j = 0; j < a.hd; j++) { const long long kj = kk[j]; d0 += qa[j] * kj; d1 += qb[j] * kj; }
            }
            sc[2 * pr] = ((d0 >> a.fa) * a.inv_sqrt) >> a.fa;
            if (two) sc[2 * pr + 1] = ((d1 >> a.fa) * a.inv_sqrt) >> a.fa;
        }
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
        if (r_lo + u >= r_hi) break;
        long long m = sc[u];
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s2));
        if (lane == 0 && m != INT64_MIN) atomicMax(&s_max[r_lo + u], m);
    }
    __syncthreads();
    if (tid < rep && s_max[tid] != INT64_MIN) atomicMax(a.hmax + kv * rep + tid, s_max[tid]);
    grid.sync();
    // ---- pass 2: exponentials (kept in registers) and their sum ---------------------------------------------------------
    unsigned ev[4] = {0, 0, 0, 0};
#pragma unroll
    for (int u = 0; u < 4; u++) {
        if (r_lo + u >= r_hi) break;
        unsigned long long e = 0;
        if (key < nk) {
            long long dlt = __ldcg(a.hmax + kv * rep + r_lo + u) - sc[u];
            dlt = dlt < a.clip ? dlt : a.clip;
            e = (unsigned long long)exp2_neg_fixed((dlt * a.log2e) >> a.fa, a.fa);
            ev[u] = (unsigned)e;
        }
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) e += __shfl_xor_sync(0xffffffffu, e, s2);
        if (lane == 0 && e) atomicAdd(&s_z[r_lo + u], e);
    }
    __syncthreads();
    if (tid < rep && s_z[tid]) atomicAdd(a.Z + kv * rep + tid, s_z[tid]);
    grid.sync();
    // ---- pass 3: probabilities into shared memory, then probabilities x values ------------------------------------------
    for (int i = tid; i < AT_MAXREP * AT_CH; i += blockDim.x) s_p[i] = 0;
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 4; u++) {
        if (r_lo + u >= r_hi) break;
        if (key < nk) {
            const unsigned long long z = __ldcg(a.Z + kv * rep + r_lo + u);
            s_p[key * AT_MAXREP + r_lo + u] = z ? (int32_t)(((unsigned long long)ev[u] << a.fa) / z) : 0;
        }
    }
    __syncthreads();
    const int G = blockDim.x / a.hd, grp = tid / a.hd, d = tid - grp * a.hd;
    long long *part = a.partial + ((long long)blockIdx.x * a.Hkv + kv) * rep * a.hd;      // this CTA's [rep][hd] partial sums
    if (grp < G) {
        for (int r0 = grp * 4; r0 < rep; r0 += G * 4) {
            long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
            for (int j = 0; j < nk; j++) {
                const int32_t v = sv[j * a.hd + d];
                const int4 p4 = *reinterpret_cast<const int4 *>(s_p + j * AT_MAXREP + r0);
                c0 += (long long)p4.x * v; c1 += (long long)p4.y * v; c2 += (long long)p4.z * v; c3 += (long long)p4.w * v;
            }
            const long long cs[4] = {c0, c1, c2, c3};
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u < rep) part[(r0 + u) * a.hd + d] = cs[u];
        }
    }
    if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0 && a.out_nl) *a.out_nl = 1;
    grid.sync();
    // ---- pass 4: every output is the sum of the chunk partials; sixteen lanes share one output ---------------------------
    if (blockIdx.x == 0 && blockIdx.y == 0)
        for (int i = tid; i < a.H; i += blockDim.x) { a.hmax[i] = INT64_MIN; a.Z[i] = 0ULL; }     // nobody reads them any more
    const long long n = (long long)a.H * a.hd;
    const int used = (int)((a.pos - a.lo) / AT_CH) + 1;                      // chunks that held keys
    const long long gid = ((long long)(blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + tid);
    const long long n_groups = (long long)gridDim.x * gridDim.y * blockDim.x / 16;
    const int sub = (int)(gid & 15);
    int nl = 1;
    bool over = false;
    // n and n_groups are even and a warp holds the two outputs 2w, 2w + 1: the bound on the even one keeps the trip count
    // uniform over the warp, as the full-mask shuffles below require
    for (long long o = gid >> 4; (o & ~1LL) < n; o += n_groups) {
        long long sum = 0;
        if (o < n) {
            const int h = (int)(o / a.hd), dd = (int)(o - (long long)h * a.hd), kvh = h / rep, r = h - kvh * rep;
            for (int c = sub; c < used; c += 16)
                sum += __ldcg(a.partial + (((long long)c * a.Hkv + kvh) * rep + r) * a.hd + dd);
        }
#pragma unroll
        for (int s2 = 8; s2 > 0; s2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s2);
        if (o < n && sub == 0) {
            const long long y = sum >> a.fa;
            if (a.out) a.out[o] = y;
            if (a.out_limbs) {
                bool ok;
                const uint64_t dg = balanced_digits8(y, ok);
                over |= !ok;
                nl = max(nl, digits_used(dg));
#pragma unroll
                for (int l = 0; l < 8; l++) a.out_limbs[l * n + o] = (int8_t)(dg >> (8 * l));
            }
        }
    }
    if (over) atomicOr(a.flags, 1);
    if (a.out_limbs && a.out_nl && nl > 1) atomicMax(a.out_nl, nl);
}

// ---- the same four passes with one CTA per SM (up to 148 CTAs of 512 threads instead of 256 of 256) ------------------
// Every KV head's visible keys are cut into as many chunks as there are SMs per head, so each SM holds exactly one
// CTA, the grid barriers have fewer participants and the per-chunk partial sums are fewer.  The K and V rows of a
// chunk arrive through bulk copies requested at kernel entry (V lands while the scores and the exponentials are
// computed); scores are register-tiled (a lane owns one key and a quarter of the head dimension for all query heads of
// the KV head, so a key value is read from shared memory once for eight heads) and so is probability x value (a
// thread owns two output dimensions of four heads for a quarter of the keys).
constexpr int AF_THREADS = 512;
constexpr int AF_HEADS = 8;                  // query heads per KV head this form carries
constexpr int TS_CHUNKS_MIN = 4, TS_CHUNKS_MAX = 16;      // 64-key chunks one CTA of attn_scores_tc_kernel walks (a.chunk, chosen at launch)
constexpr unsigned AF_POLLS = 1u << 22;

__device__ __forceinline__ uint32_t af_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool af_wait(uint64_t *bar) {
    for (unsigned it = 0; it < AF_POLLS; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(af_u32(bar)) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void af_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(af_u32(dst)), "l"(src), "r"(bytes), "r"(af_u32(bar)) : "memory");
}

// the four bytes of four consecutive int32 values, transposed: d_b = byte b of (x, y, z, w)
__device__ __forceinline__ void af_bytes(const int4 v, uint32_t &d0, uint32_t &d1, uint32_t &d2, uint32_t &d3) {
    const uint32_t t0 = __byte_perm((uint32_t)v.x, (uint32_t)v.y, 0x5140), t1 = __byte_perm((uint32_t)v.x, (uint32_t)v.y, 0x7362);
    const uint32_t t2 = __byte_perm((uint32_t)v.z, (uint32_t)v.w, 0x5140), t3 = __byte_perm((uint32_t)v.z, (uint32_t)v.w, 0x7362);
    d0 = __byte_perm(t0, t2, 0x5410); d1 = __byte_perm(t0, t2, 0x7632);
    d2 = __byte_perm(t1, t3, 0x5410); d3 = __byte_perm(t1, t3, 0x7632);
}
// D(16x8,s32) += A(16x32, 8-bit, row) * B(32x8, 8-bit, col) with the signedness of each operand chosen per byte plane
template <bool A_SIGNED, bool B_SIGNED>
__device__ __forceinline__ void af_mma(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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

// Barrier among the CTAs of one KV head (the row maximum and the normaliser are per head, so nothing wider is needed): a
// counter that only grows within a launch, `target` arrivals open it.  The launch is cooperative, so every CTA is resident;
// the wait is bounded all the same and reports a give-up instead of spinning on.  The last CTA of the launch zeroes the counter.
__device__ __forceinline__ bool af_group_barrier(unsigned *counter, unsigned target) {
    __shared__ int s_open;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        unsigned seen = 0;
        for (int spin = 0; spin < (1 << 22); spin++) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= target) break;
        }
        s_open = seen >= target ? 1 : 0;
    }
    __syncthreads();
    return s_open != 0;
}

__global__ void __launch_bounds__(AF_THREADS, 1) attn_fat_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }          // uniform over the grid
    extern __shared__ __align__(16) unsigned char af_smem[];
    __shared__ long long s_max[AF_HEADS];
    __shared__ unsigned long long s_z[AF_HEADS];
    __shared__ int s_wide, s_timeout, s_last, s_nl_out;
    __shared__ __align__(8) uint64_t bars[2];
    const int C = a.chunk, hd = a.hd, rep = a.H / a.Hkv, kv = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, half = hd / 2;
    const int KQ = AF_THREADS / hd;                                         // key groups of the probability x value pass
    // Key and value rows lie in groups of eight consecutive rows, as in the cache, so one bulk copy brings a group; a gap
    // after every group (16 words for keys, 8 for values) spreads the rows that one shared-memory read touches over the banks:
    // a key read takes rows of two neighbouring groups per quarter warp, a value read rows of four groups per warp.
    auto koff = [hd](int r) { return (size_t)r * hd + (size_t)(r >> 3) * 16; };
    auto voff = [hd](int r) { return (size_t)r * hd + (size_t)(r >> 3) * 8; };
    int32_t *sk = reinterpret_cast<int32_t *>(af_smem);                     // keys, C rows
    int32_t *sv = sk + koff(C);                                             // values, C rows
    int32_t *q32 = sv + voff(C);                                            // rotated queries [8][hd] (rows beyond rep are zero)
    long long *q64 = reinterpret_cast<long long *>(q32 + AF_HEADS * hd);    // the same as int64
    unsigned *s_e = reinterpret_cast<unsigned *>(q64 + AF_HEADS * hd);      // exponentials, then probabilities [C][8]
    long long *red = reinterpret_cast<long long *>(s_e + (size_t)C * AF_HEADS);   // [KQ][8][hd] partial sums of pass 3; before that the
                                                                                  // dot products [2][C][8] of pass 1
    const int qld = hd + 16;                                                // row stride of a byte plane (bytes): heads on different banks
    int8_t *qd = reinterpret_cast<int8_t *>(red + (size_t)KQ * AF_HEADS * hd);    // bytes of the rotated queries [4][8][hd + 16]
    const int pld = C + 16;                                                 // row stride of a probability byte plane
    uint8_t *pT = reinterpret_cast<uint8_t *>(qd + 4 * AF_HEADS * qld);     // bytes of the probabilities [3][8][C + 16]
    const long long l0 = a.lo + (long long)blockIdx.x * C, l1 = min(l0 + C, a.pos + 1);
    const int nk = (int)max(0LL, l1 - l0);
    const bool own = l0 <= a.pos && a.pos < l0 + C;                         // this chunk ends with the new token's row
    const int nk_old = own ? nk - 1 : nk;                                   // rows that are already in the cache
    if (tid == 0) {
        s_wide = 0; s_timeout = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(af_u32(&bars[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(af_u32(&bars[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint32_t bytes = (uint32_t)((size_t)nk_old * hd * 4);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(af_u32(&bars[0])), "r"(bytes) : "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(af_u32(&bars[1])), "r"(bytes) : "memory");
    }
    if (tid < AF_HEADS) { s_max[tid] = INT64_MIN; s_z[tid] = 0ULL; }
    __syncthreads();
    // key rows below the new position were written by earlier steps: requested before the dependency wait
    // (one copy per group of eight rows: the copy unit takes a dozen clocks per request, whatever its size)
    for (int r = 8 * tid; r < nk_old; r += 8 * AF_THREADS)
        af_copy(sk + koff(r), a.kcache + ((long long)kv * a.Lmax + l0 + r) * hd, (uint32_t)(min(8, nk_old - r) * hd * 4), &bars[0]);
    if (a.pdl) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }
    // ---- rotated queries ------------------------------------------------------------------------------------------------
    bool wide = false;
    for (int idx = tid; idx < AF_HEADS * half; idx += AF_THREADS) {
        const int r = idx / half, i = idx - r * half;
        const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
        int64_t x0 = 0, x1 = 0;
        if (r < rep) {
            const int64_t *src = a.q + (long long)(kv * rep + r) * hd;
            x0 = src[i0]; x1 = src[i1];
            at_rotate(a, a.pos, i, x0, x1);
        }
        q64[r * hd + i0] = x0; q64[r * hd + i1] = x1;
        q32[r * hd + i0] = (int32_t)x0; q32[r * hd + i1] = (int32_t)x1;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            qd[(b * AF_HEADS + r) * qld + i0] = (int8_t)((uint32_t)(int32_t)x0 >> (8 * b));
            qd[(b * AF_HEADS + r) * qld + i1] = (int8_t)((uint32_t)(int32_t)x1 >> (8 * b));
        }
        wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
    }
    // the value rows are asked for once the key rows have had the memory system to themselves for a while (they are needed
    // only after two barriers)
    for (int r = 8 * (tid - AF_THREADS / 2); r >= 0 && r < nk_old; r += 8 * AF_THREADS)   // the upper half of the CTA asks for the value rows
        af_copy(sv + voff(r), a.vcache + ((long long)kv * a.Lmax + l0 + r) * hd, (uint32_t)(min(8, nk_old - r) * hd * 4), &bars[1]);
    if (wide) s_wide = 1;
    if (own) {                                                              // the new token's row: cache and shared memory
        bool bad = false;
        for (int i = tid; i < half; i += AF_THREADS) {
            const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
            int64_t x0 = a.k[kv * hd + i0], x1 = a.k[kv * hd + i1];
            at_rotate(a, a.pos, i, x0, x1);
            bad |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
            int32_t *dst = a.kcache + ((long long)kv * a.Lmax + a.pos) * hd;
            dst[i0] = (int32_t)x0; dst[i1] = (int32_t)x1;
            sk[koff(nk - 1) + i0] = (int32_t)x0; sk[koff(nk - 1) + i1] = (int32_t)x1;
        }
        for (int i = tid; i < hd; i += AF_THREADS) {
            const int64_t v = a.v[kv * hd + i];
            bad |= v != (int32_t)v;
            a.vcache[((long long)kv * a.Lmax + a.pos) * hd + i] = (int32_t)v;
            sv[voff(nk - 1) + i] = (int32_t)v;
        }
        if (bad) atomicOr(a.flags, 4);
    }
    if (!af_wait(&bars[0])) s_timeout = 1;
    __syncthreads();
    // ---- pass 1 on the tensor cores: an int32 is its four bytes, x = b0 + 2^8 b1 + 2^16 b2 + 2^24 b3 with b0..b2 unsigned and b3
    //      signed, so q . k = sum over byte pairs of 2^(8(a+b)) (k_a . q_b), every pair an exact int8 MMA (16 keys x 8 heads x 32
    //      dimensions), pairs of equal a + b sharing an int32 accumulator (at most 4 x 255^2 x hd < 2^31).  Two warps share a
    //      16-key tile, half of the head dimension each, where there are at most eight tiles.
    const bool use_wide = s_wide != 0;
    long long *dots = red;
    const int tiles_c = C >> 4, ksteps = hd / 32;
    const bool split = tiles_c <= 8 && (ksteps & 1) == 0;
    if (!use_wide) {
        const int kt = split ? (warp >> 1) : warp, kh = split ? (warp & 1) : 0;
        const int s_lo = split ? kh * (ksteps / 2) : 0, s_hi = split ? s_lo + ksteps / 2 : ksteps;
        if (kt < tiles_c && kt * 16 < nk) {                                 // warp-uniform
            int acc[7][4];
#pragma unroll
            for (int i = 0; i < 7; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0; }
            const int g = lane >> 2, t = lane & 3;
            // fragment row g is key (g & 1) * 8 + (g >> 1) of the tile and row g + 8 the key four further on: the two rows
            // of a quarter warp then lie in neighbouring groups, half the banks apart
            const int keyA = kt * 16 + (g & 1) * 8 + (g >> 1);
            const int32_t *rowA = sk + koff(keyA), *rowB = rowA + 4 * hd;
            for (int st = s_lo; st < s_hi; st++) {
                uint32_t A[4][4];
                af_bytes(*reinterpret_cast<const int4 *>(rowA + 32 * st + 4 * t), A[0][0], A[1][0], A[2][0], A[3][0]);
                af_bytes(*reinterpret_cast<const int4 *>(rowB + 32 * st + 4 * t), A[0][1], A[1][1], A[2][1], A[3][1]);
                af_bytes(*reinterpret_cast<const int4 *>(rowA + 32 * st + 16 + 4 * t), A[0][2], A[1][2], A[2][2], A[3][2]);
                af_bytes(*reinterpret_cast<const int4 *>(rowB + 32 * st + 16 + 4 * t), A[0][3], A[1][3], A[2][3], A[3][3]);
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int8_t *qb = qd + (b * AF_HEADS + g) * qld + 32 * st + 4 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(qb), b1 = *reinterpret_cast<const uint32_t *>(qb + 16);
#pragma unroll
                    for (int aa = 0; aa < 4; aa++) {
                        if (aa < 3 && b < 3) af_mma<false, false>(acc[aa + b], A[aa], b0, b1);
                        else if (aa < 3) af_mma<false, true>(acc[aa + b], A[aa], b0, b1);
                        else if (b < 3) af_mma<true, false>(acc[aa + b], A[aa], b0, b1);
                        else af_mma<true, true>(acc[aa + b], A[aa], b0, b1);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                long long dot = 0;
#pragma unroll
                for (int w = 6; w >= 0; w--) dot = dot * 256 + (long long)acc[w][i];
                const int row = keyA + (i >= 2 ? 4 : 0), col = 2 * t + (i & 1);
                dots[((size_t)kh * C + row) * AF_HEADS + col] = dot;
            }
        }
    } else {
        // a query value beyond int32: wrapping 64-bit products, one (key, head) pair per thread and turn
        for (int i = tid; i < nk * AF_HEADS; i += AF_THREADS) {
            const int key = i >> 3, h = i & 7;
            long long dot = 0;
            if (h < rep) {
                const int32_t *kk = sk + koff(key);
                for (int j = 0; j < hd; j++) dot += q64[h * hd + j] * (long long)kk[j];
            }
            dots[i] = dot;
        }
    }
    __syncthreads();
    // scores of the (key, head) pairs i = tid, tid + 512, ...: key = i / 8, head = i % 8 = lane % 8
    const int head = lane & 7;
    long long sc[4] = {INT64_MIN, INT64_MIN, INT64_MIN, INT64_MIN};
    long long mloc = INT64_MIN;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = tid + u * AF_THREADS;
        if (i < nk * AF_HEADS && head < rep) {
            long long d = dots[i];
            if (split && !use_wide) d += dots[(size_t)C * AF_HEADS + i];
            sc[u] = ((d >> a.fa) * a.inv_sqrt) >> a.fa;
            mloc = max(mloc, sc[u]);
        }
    }
    mloc = max(mloc, __shfl_xor_sync(0xffffffffu, mloc, 8));
    mloc = max(mloc, __shfl_xor_sync(0xffffffffu, mloc, 16));
    if (lane < 8 && mloc != INT64_MIN) atomicMax(&s_max[head], mloc);
    __syncthreads();
    if (tid < rep && s_max[tid] != INT64_MIN) atomicMax(a.hmax + kv * rep + tid, s_max[tid]);
    if (!af_group_barrier(a.ticket + 1 + kv, gridDim.x)) s_timeout = 1;
    // ---- pass 2: exponentials into shared memory and their sums ------------------------------------------------------------
    unsigned long long zloc = 0ULL;
    const long long hm = head < rep ? __ldcg(a.hmax + kv * rep + head) : 0;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = tid + u * AF_THREADS;
        if (i >= nk * AF_HEADS) continue;
        unsigned e = 0;
        if (head < rep) {
            long long dlt = hm - sc[u];
            dlt = dlt < a.clip ? dlt : a.clip;
            e = (unsigned)exp2_neg_fixed((dlt * a.log2e) >> a.fa, a.fa);
            zloc += e;
        }
        s_e[i] = e;
    }
    zloc += __shfl_xor_sync(0xffffffffu, zloc, 8);
    zloc += __shfl_xor_sync(0xffffffffu, zloc, 16);
    if (lane < 8 && zloc) atomicAdd(&s_z[head], zloc);
    __syncthreads();
    if (tid < rep && s_z[tid]) atomicAdd(a.Z + kv * rep + tid, s_z[tid]);
    if (!af_group_barrier(a.ticket + 1 + kv, 2u * gridDim.x)) s_timeout = 1;
    // ---- pass 3: probabilities as byte planes, then probabilities x values on the tensor cores ---------------------------
    //      out[head][dim] = sum over keys p[key][head] v[key][dim]: A = bytes of p (heads x keys; p <= 2^fa has three unsigned
    //      bytes), B = bytes of v gathered from four key rows (keys x dims), a warp owns eight dimensions for all keys
    const int nk32 = (nk + 31) & ~31;
    // a thread's pairs all belong to head tid % 8: one reciprocal of that head's normaliser, then floor(e 2^fa / z) per pair
    // as a high product with an exact fix-up instead of a 64-bit division each
    const unsigned long long z_own = head < rep ? __ldcg(a.Z + kv * rep + head) : 0ULL;
    const unsigned long long z_inv = recip_below(z_own);
    for (int idx = tid; idx < nk32 * AF_HEADS; idx += AF_THREADS) {
        const int key = idx >> 3, h = idx & (AF_HEADS - 1);
        unsigned p = 0;
        if (key < nk && z_own) {
            const unsigned long long n = (unsigned long long)s_e[idx] << a.fa;
            unsigned long long q = __umul64hi(n, z_inv), r = n - q * z_own;
            while (r >= z_own) { q++; r -= z_own; }
            p = (unsigned)q;
        }
        // position of the key inside its 32-key step: keys 8t + 4u + j sit at 16u + 4t + j, so that the four rows a lane
        // gathers for one step come from four different groups of the value rows
        const int kpos = (key & ~31) | ((key & 4) << 2) | ((key & 24) >> 1) | (key & 3);
#pragma unroll
        for (int b = 0; b < 3; b++) pT[(b * AF_HEADS + h) * pld + kpos] = (uint8_t)(p >> (8 * b));
    }
    // value rows beyond the chunk's keys multiply zero probabilities but must hold numbers: clear them
    for (int i = tid; i < (nk32 - nk) * hd; i += AF_THREADS) sv[voff(nk + i / hd) + (i % hd)] = 0;
    if (!af_wait(&bars[1])) s_timeout = 1;
    __syncthreads();
    long long *accum = a.acc + (long long)kv * rep * hd;                                  // the [rep][hd] sums of this KV head, shared by its chunks
    {
        const int g = lane >> 2, t = lane & 3;
        for (int nt = warp; nt < hd / 8; nt += AF_THREADS / 32) {           // eight dimensions per warp and turn
            int acc[6][4];
#pragma unroll
            for (int i = 0; i < 6; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0; }
            for (int st = 0; st < nk32 / 32; st++) {
                uint32_t B0[4], B1[4];
                const int32_t *vb = sv + voff(32 * st + 8 * t) + nt * 8 + g;          // positions 4t + j and 16 + 4t + j: keys 8t + j, 8t + 4 + j
                af_bytes(make_int4(vb[0], vb[hd], vb[2 * hd], vb[3 * hd]), B0[0], B0[1], B0[2], B0[3]);
                af_bytes(make_int4(vb[4 * hd], vb[5 * hd], vb[6 * hd], vb[7 * hd]), B1[0], B1[1], B1[2], B1[3]);
#pragma unroll
                for (int pa = 0; pa < 3; pa++) {
                    const uint8_t *pp = pT + (pa * AF_HEADS + g) * pld + 32 * st + 4 * t;
                    const uint32_t A[4] = {*reinterpret_cast<const uint32_t *>(pp), 0u, *reinterpret_cast<const uint32_t *>(pp + 16), 0u};
#pragma unroll
                    for (int vb8 = 0; vb8 < 4; vb8++) {
                        if (vb8 < 3) af_mma<false, false>(acc[pa + vb8], A, B0[vb8], B1[vb8]);
                        else af_mma<false, true>(acc[pa + vb8], A, B0[vb8], B1[vb8]);
                    }
                }
            }
            // rows 0..7 of the tile are the heads: c0, c1 = (head g, dims 2t, 2t + 1)
#pragma unroll
            for (int i = 0; i < 2; i++) {
                long long sum = 0;
#pragma unroll
                for (int w = 5; w >= 0; w--) sum = sum * 256 + (long long)acc[w][i];
                if (g < rep) atomicAdd(reinterpret_cast<unsigned long long *>(accum + g * hd + nt * 8 + 2 * t + i), (unsigned long long)sum);
            }
        }
    }
    // ---- the chunk sums were added into one accumulator per output (integer adds are order-free); of every KV head the CTA
    //      that arrives last (a counter, no waiting) shifts its heads' sums, writes them and their digit planes, leaves the
    //      digit count of its part in out_nl[kv] and returns the statistics and counters of the head to their initial state.
    //      That spares a third barrier and a reduction over the chunks, and the four read-outs run side by side.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const bool last = atomicAdd(a.ticket + 1 + gridDim.y + kv, 1u) == gridDim.x - 1;
        if (last) __threadfence();
        s_last = last ? 1 : 0; s_nl_out = 1;
    }
    __syncthreads();
    if (s_timeout && tid == 0) atomicOr(a.flags, 8);
    if (!s_last) return;
    const long long n = (long long)a.H * hd, base = (long long)kv * rep * hd;      // plane stride; this head's first output
    const int cnt = rep * hd;                                               // a multiple of 32
    int nl = 1;
    bool over = false;
    const bool word_planes = (reinterpret_cast<uintptr_t>(a.out_limbs) & 3) == 0;
    for (int q = tid * 4; q < cnt; q += AF_THREADS * 4) {                   // four consecutive outputs per thread and turn
        const long long i = base + q;
        const longlong2 v0 = __ldcg(reinterpret_cast<const longlong2 *>(a.acc + i));
        const longlong2 v1 = __ldcg(reinterpret_cast<const longlong2 *>(a.acc + i + 2));
        const long long y[4] = {v0.x >> a.fa, v0.y >> a.fa, v1.x >> a.fa, v1.y >> a.fa};
        if (a.out) { a.out[i] = y[0]; a.out[i + 1] = y[1]; a.out[i + 2] = y[2]; a.out[i + 3] = y[3]; }
        if (a.out_limbs) {
            uint64_t dg[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                bool ok;
                dg[e] = balanced_digits8(y[e], ok);
                over |= !ok;
                nl = max(nl, digits_used(dg[e]));
            }
            uint32_t pw[8];                                                  // word l = digit l of the four outputs (a byte transpose)
#pragma unroll
            for (int hw = 0; hw < 2; hw++) {
                const uint32_t w0 = (uint32_t)(dg[0] >> (32 * hw)), w1 = (uint32_t)(dg[1] >> (32 * hw));
                const uint32_t w2 = (uint32_t)(dg[2] >> (32 * hw)), w3 = (uint32_t)(dg[3] >> (32 * hw));
                const uint32_t lo01 = __byte_perm(w0, w1, 0x5140), hi01 = __byte_perm(w0, w1, 0x7362);
                const uint32_t lo23 = __byte_perm(w2, w3, 0x5140), hi23 = __byte_perm(w2, w3, 0x7362);
                pw[4 * hw + 0] = __byte_perm(lo01, lo23, 0x5410); pw[4 * hw + 1] = __byte_perm(lo01, lo23, 0x7632);
                pw[4 * hw + 2] = __byte_perm(hi01, hi23, 0x5410); pw[4 * hw + 3] = __byte_perm(hi01, hi23, 0x7632);
            }
            if (word_planes) {
#pragma unroll
                for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(a.out_limbs + l * n + i) = pw[l];
            } else {
#pragma unroll
                for (int l = 0; l < 8; l++)
                    for (int e = 0; e < 4; e++) a.out_limbs[l * n + i + e] = (int8_t)(pw[l] >> (8 * e));
            }
        }
        *reinterpret_cast<longlong2 *>(a.acc + i) = make_longlong2(0, 0);
        *reinterpret_cast<longlong2 *>(a.acc + i + 2) = make_longlong2(0, 0);
    }
    if (over) atomicOr(a.flags, 1);
    if (a.out_limbs) atomicMax(&s_nl_out, nl);
    if (tid < rep) { a.hmax[kv * rep + tid] = INT64_MIN; a.Z[kv * rep + tid] = 0ULL; }
    __syncthreads();
    if (tid == 0) {
        a.ticket[1 + kv] = 0u; a.ticket[1 + gridDim.y + kv] = 0u;          // this head's barrier counter and its ticket
        if (a.out_nl) a.out_nl[kv] = s_nl_out;
    }
}

// ---- several tokens at once (a prefill chunk, or the new tokens of independent sequences): the scores on the tensor cores,
//      byte decomposition as in attn_fat_kernel.  Same grid as attn_scores_kernel, which remains for shapes this does not
//      carry (more than eight query heads per KV head, head_dim other than 64 / 128).
__global__ void __launch_bounds__(256) attn_scores_tc_kernel(const AttnArgs a_in) {
    AttnArgs a = a_in;
    if (!at_span(a_in, a.pos, a.lo)) { at_refuse(a_in); return; }
    at_batch(a);
    const long long Ls = a.Ls ? a.Ls : a.Lmax;
    extern __shared__ __align__(16) unsigned char ts_smem[];
    __shared__ long long s_max[AF_HEADS];
    __shared__ int s_wide, s_q24;
    const int kv = blockIdx.y, rep = a.H / a.Hkv, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, hd = a.hd, half = hd / 2;
    const int ld = hd + 4, qld = hd + 16;
    // a CTA walks a.chunk consecutive 64-key chunks: the queries are rotated once and the next chunk's keys stream in
    // (cp.async into the other buffer) while the current chunk is multiplied
    const int walk = a.chunk;
    const long long first = a.lo + (long long)blockIdx.x * walk * AT_CH;
    if (first > a.pos) return;                             // all of this CTA's chunks lie past the token's position
    long long *q64 = reinterpret_cast<long long *>(ts_smem);                 // [8][hd]
    long long *dots = q64 + AF_HEADS * hd;                                  // [2][64][8]
    int32_t *skb = reinterpret_cast<int32_t *>(dots + 2 * AT_CH * AF_HEADS); // two key buffers [64][hd + 4]
    int8_t *qd = reinterpret_cast<int8_t *>(skb + 2 * AT_CH * ld);          // [4][8][hd + 16]
    if (tid == 0) { s_wide = 0; s_q24 = 0; }
    if (tid < AF_HEADS) s_max[tid] = INT64_MIN;
    const int vec_per_row = hd / 4;
    auto request = [&](int c) {                            // keys of chunk c of this CTA into buffer c & 1
        const long long l0 = first + (long long)c * AT_CH;
        const int nk = (int)max(0LL, min(l0 + AT_CH, a.pos + 1) - l0);
        const int4 *src = reinterpret_cast<const int4 *>(a.kcache + ((long long)kv * a.Lmax + l0) * hd);
        int32_t *dst = skb + (size_t)(c & 1) * AT_CH * ld;
        for (int i = tid; i < nk * vec_per_row; i += blockDim.x) {
            const int row = i / vec_per_row;
            const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + row * ld + (i - row * vec_per_row) * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    request(0);
    __syncthreads();
    bool wide = false, wide24 = false;
    for (int idx = tid; idx < AF_HEADS * half; idx += blockDim.x) {
        const int r = idx / half, i = idx - r * half;
        const int i0 = a.rope == 2 ? i : 2 * i, i1 = a.rope == 2 ? i + half : 2 * i + 1;
        int64_t x0 = 0, x1 = 0;
        if (r < rep) {
            const int64_t *src = a.q + (long long)(kv * rep + r) * hd;
            x0 = src[i0]; x1 = src[i1];
            at_rotate(a, a.pos, i, x0, x1);
        }
        q64[r * hd + i0] = x0; q64[r * hd + i1] = x1;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            qd[(b * AF_HEADS + r) * qld + i0] = (int8_t)((uint32_t)(int32_t)x0 >> (8 * b));
            qd[(b * AF_HEADS + r) * qld + i1] = (int8_t)((uint32_t)(int32_t)x1 >> (8 * b));
        }
        wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
        wide24 |= x0 < -(1 << 23) || x0 >= (1 << 23) || x1 < -(1 << 23) || x1 >= (1 << 23);
    }
    if (wide) s_wide = 1;
    if (wide24) s_q24 = 1;
    __syncthreads();
    const bool use_wide = s_wide != 0, q_narrow = s_q24 == 0;
    const int ksteps = hd / 32;
    const bool split = (ksteps & 1) == 0;                  // four 16-key tiles: two warps per tile, half of the head dimension each
    const int key = tid & (AT_CH - 1);                     // thread -> (key, heads tid / 64 and tid / 64 + 4) for the score stores
    long long mloc[2] = {INT64_MIN, INT64_MIN};
    for (int c = 0; c < walk; c++) {
        const long long l0 = first + (long long)c * AT_CH;
        if (l0 > a.pos) break;                             // uniform over the CTA
        const int nk = (int)(min(l0 + AT_CH, a.pos + 1) - l0);
        const bool more = c + 1 < walk && l0 + AT_CH <= a.pos;
        if (more) { request(c + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                   // chunk c has landed for every thread
        const int32_t *sk = skb + (size_t)(c & 1) * AT_CH * ld;
        if (!use_wide) {
            const int kt = split ? (warp >> 1) : warp, kh = split ? (warp & 1) : 0;
            const int s_lo = split ? kh * (ksteps / 2) : 0, s_hi = split ? s_lo + ksteps / 2 : ksteps;
            if (kt < AT_CH / 16 && kt * 16 < nk) {
                int acc[7][4];
#pragma unroll
                for (int i = 0; i < 7; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0; }
                const int g = lane >> 2, t = lane & 3;
                const int32_t *rowA = sk + (size_t)(kt * 16 + g) * ld, *rowB = rowA + 8 * ld;
                for (int st = s_lo; st < s_hi; st++) {
                    uint32_t A[4][4];
                    const int4 k0 = *reinterpret_cast<const int4 *>(rowA + 32 * st + 4 * t), k1 = *reinterpret_cast<const int4 *>(rowB + 32 * st + 4 * t);
                    const int4 k2 = *reinterpret_cast<const int4 *>(rowA + 32 * st + 16 + 4 * t), k3 = *reinterpret_cast<const int4 *>(rowB + 32 * st + 16 + 4 * t);
                    af_bytes(k0, A[0][0], A[1][0], A[2][0], A[3][0]);
                    af_bytes(k1, A[0][1], A[1][1], A[2][1], A[3][1]);
                    af_bytes(k2, A[0][2], A[1][2], A[2][2], A[3][2]);
                    af_bytes(k3, A[0][3], A[1][3], A[2][3], A[3][3]);
                    // keys and queries within [-2^23, 2^23): three byte planes each, the third signed (9 byte pairs instead of
                    // 16); decided per warp and K step, the accumulators take either form
                    auto fits = [](const int4 v) {
                        return ((unsigned)(v.x + (1 << 23)) | (unsigned)(v.y + (1 << 23)) | (unsigned)(v.z + (1 << 23)) | (unsigned)(v.w + (1 << 23))) < (1u << 24);
                    };
                    const bool narrow = q_narrow && __all_sync(0xffffffffu, fits(k0) && fits(k1) && fits(k2) && fits(k3));
                    if (narrow) {
#pragma unroll
                        for (int b = 0; b < 3; b++) {
                            const int8_t *qb = qd + (b * AF_HEADS + g) * qld + 32 * st + 4 * t;
                            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(qb), b1 = *reinterpret_cast<const uint32_t *>(qb + 16);
#pragma unroll
                            for (int aa = 0; aa < 3; aa++) {
                                if (aa < 2 && b < 2) af_mma<false, false>(acc[aa + b], A[aa], b0, b1);
                                else if (aa < 2) af_mma<false, true>(acc[aa + b], A[aa], b0, b1);
                                else if (b < 2) af_mma<true, false>(acc[aa + b], A[aa], b0, b1);
                                else af_mma<true, true>(acc[aa + b], A[aa], b0, b1);
                            }
                        }
                    } else {
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        const int8_t *qb = qd + (b * AF_HEADS + g) * qld + 32 * st + 4 * t;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(qb), b1 = *reinterpret_cast<const uint32_t *>(qb + 16);
#pragma unroll
                        for (int aa = 0; aa < 4; aa++) {
                            if (aa < 3 && b < 3) af_mma<false, false>(acc[aa + b], A[aa], b0, b1);
                            else if (aa < 3) af_mma<false, true>(acc[aa + b], A[aa], b0, b1);
                            else if (b < 3) af_mma<true, false>(acc[aa + b], A[aa], b0, b1);
                            else af_mma<true, true>(acc[aa + b], A[aa], b0, b1);
                        }
                    }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    long long dot = 0;
#pragma unroll
                    for (int w = 6; w >= 0; w--) dot = dot * 256 + (long long)acc[w][i];
                    const int row = kt * 16 + g + (i >= 2 ? 8 : 0), col = 2 * t + (i & 1);
                    dots[((size_t)kh * AT_CH + row) * AF_HEADS + col] = dot;
                }
            }
        } else {
            for (int i = tid; i < nk * AF_HEADS; i += blockDim.x) {         // a query value beyond int32: wrapping 64-bit products
                const int kk2 = i >> 3, h = i & 7;
                long long dot = 0;
                if (h < rep) {
                    const int32_t *kk = sk + (size_t)kk2 * ld;
                    for (int j = 0; j < hd; j++) dot += q64[h * hd + j] * (long long)kk[j];
                }
                dots[i] = dot;
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int h = (tid >> 6) + 4 * u;
            if (key < nk && h < rep) {
                long long d = dots[key * AF_HEADS + h];
                if (split && !use_wide) d += dots[(size_t)(AT_CH + key) * AF_HEADS + h];
                const long long sc = ((d >> a.fa) * a.inv_sqrt) >> a.fa;
                a.scores[(long long)(kv * rep + h) * Ls + l0 + key] = sc;
                mloc[u] = max(mloc[u], sc);
            }
        }
        __syncthreads();                                   // dots and the buffer of chunk c may be overwritten
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int h = (tid >> 6) + 4 * u;
        long long m = mloc[u];
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s2));
        if (lane == 0 && m != INT64_MIN && h < rep) atomicMax(&s_max[h], m);
    }
    __syncthreads();
    if (tid < rep && s_max[tid] != INT64_MIN) atomicMax(a.hmax + kv * rep + tid, s_max[tid]);
}

// one row of a registered Q4_K / Q6_K matrix as int64 at 2^frac (the embedding look-up)
// (grid.y rows at once: row_dev[y] -> out[y][nb * 256])
__global__ void embed_row_kernel(const uint8_t *w, int qtype, long long nb, const int *row_dev, long long row_host, int frac,
                                 int64_t *out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb * 256) return;
    out += (long long)blockIdx.y * nb * 256;
    const long long o = row_dev ? (long long)row_dev[blockIdx.y] : row_host, b = i >> 8;
    const int e = (int)(i & 255);
    auto byte = [&](int k) { return (int)repacked_byte(w, qtype, nb, o, b, k); };
    int64_t val;
    if (qtype == QT_Q4K) {
        const int64_t dq = half_to_fixed(byte(0) | (byte(1) << 8), frac), dmq = half_to_fixed(byte(2) | (byte(3) << 8), frac);
        const int j = e >> 5, l = e & 31;
        int sc, mn;
        if (j < 4) { sc = byte(4 + j) & 63; mn = byte(8 + j) & 63; }
        else { sc = (byte(8 + j) & 0xF) | ((byte(j) >> 6) << 4); mn = (byte(8 + j) >> 4) | ((byte(4 + j) >> 6) << 4); }
        const int q = (byte(16 + 32 * (j >> 1) + l) >> ((j & 1) * 4)) & 0xF;
        val = dq * sc * q - dmq * mn;
    } else {
        const int64_t dq = half_to_fixed(byte(208) | (byte(209) << 8), frac);
        const int sb = e >> 4, l = e & 15, half = sb >> 3, k = (sb >> 1) & 3, l0 = (sb & 1) * 16;
        const int ql = byte(64 * half + 32 * (k & 1) + l0 + l), qh = byte(128 + 32 * half + l0 + l);
        const int q = (((k < 2) ? (ql & 0xF) : (ql >> 4)) | (((qh >> (2 * k)) & 3) << 4)) - 32;
        val = dq * (int64_t)(int8_t)byte(192 + 8 * half + 2 * k + (sb & 1)) * q;
    }
    out[i] = val;
}

// arg-max of each of grid.x rows of n values, lowest index on ties: one CTA per row
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const int64_t *x, long long n, int *out) {
    __shared__ long long s_v[32];
    __shared__ long long s_i[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t *row = x + (long long)blockIdx.x * n;
    long long bv = INT64_MIN, bi = n;
    auto better = [](long long ov, long long oi, long long v, long long i) { return ov > v || (ov == v && oi < i); };
    long long i = tid * 2LL;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0)
        for (; i + 1 < n; i += 2048) {                              // two values per load
            const longlong2 v = *reinterpret_cast<const longlong2 *>(row + i);
            if (better(v.x, i, bv, bi)) { bv = v.x; bi = i; }
            if (better(v.y, i + 1, bv, bi)) { bv = v.y; bi = i + 1; }
        }
    else
        for (; i + 1 < n; i += 2048) {
            if (better(row[i], i, bv, bi)) { bv = row[i]; bi = i; }
            if (better(row[i + 1], i + 1, bv, bi)) { bv = row[i + 1]; bi = i + 1; }
        }
    if (i < n && better(row[i], i, bv, bi)) { bv = row[i]; bi = i; }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const long long ov = __shfl_xor_sync(0xffffffffu, bv, s), oi = __shfl_xor_sync(0xffffffffu, bi, s);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = s_v[lane]; bi = s_i[lane];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const long long ov = __shfl_xor_sync(0xffffffffu, bv, s), oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (int)bi;
    }
}

// arg-max with the lowest index on ties: every CTA leaves its candidate in a static table, the CTA that arrives last
// (a counter, no waiting) picks among the candidates and clears the counter for the next launch on the stream
constexpr int AM_CTAS = 148;
__device__ long long g_am_v[AM_CTAS], g_am_i[AM_CTAS];
__device__ unsigned g_am_done;

__global__ void __launch_bounds__(1024) argmax_kernel(const int64_t *x, long long n, int *out) {
    __shared__ long long s_v[32];
    __shared__ long long s_i[32];
    __shared__ bool s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    long long bv = INT64_MIN, bi = n;
    auto better = [](long long ov, long long oi, long long v, long long i) { return ov > v || (ov == v && oi < i); };
    auto block_pick = [&]() {                                       // result valid in thread 0
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const long long ov = __shfl_xor_sync(0xffffffffu, bv, s), oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
        __syncthreads();
        if (warp == 0) {
            bv = lane < (blockDim.x >> 5) ? s_v[lane] : INT64_MIN; bi = lane < (blockDim.x >> 5) ? s_i[lane] : n;
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                const long long ov = __shfl_xor_sync(0xffffffffu, bv, s), oi = __shfl_xor_sync(0xffffffffu, bi, s);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
        }
    };
    for (long long i = (long long)blockIdx.x * blockDim.x + tid; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long v = x[i];
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    block_pick();
    if (gridDim.x == 1) { if (tid == 0) *out = (int)bi; return; }
    if (tid == 0) {
        g_am_v[blockIdx.x] = bv; g_am_i[blockIdx.x] = bi;
        __threadfence();
        s_last = atomicAdd(&g_am_done, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    bv = INT64_MIN; bi = n;
    if (tid < (int)gridDim.x) { bv = __ldcg(&g_am_v[tid]); bi = __ldcg(&g_am_i[tid]); }
    __syncthreads();                                                // s_v / s_i are reused
    block_pick();
    if (tid == 0) { *out = (int)bi; g_am_done = 0; }
}

}  // namespace

bool attn_shape_ok(int H, int Hkv, int hd) {
    const int rep = Hkv > 0 ? H / Hkv : 0;
    return !(H <= 0 || Hkv <= 0 || H % Hkv || rep > AT_MAXREP || hd < 32 || hd > 256 || hd % 32 || 256 % hd ||
             rep > (256 / hd) * (AT_MAXREP / 2));
}

cudaError_t launch_attn_decode(const AttnArgs &a, cudaStream_t s) {
    const int rep = a.Hkv > 0 ? a.H / a.Hkv : 0;
    if (!attn_shape_ok(a.H, a.Hkv, a.hd) ||
        a.pos < 0 || a.pos >= a.Lmax || a.fa < 1 || a.fa > 29 || (a.rope && (!a.cos || !a.sin)))
        return cudaErrorInvalidValue;
    // a.pos is the position itself, or with pos_dev an upper bound of it: the grids cover the largest key span
    const long long lo_min = (a.window > 0 && !a.pos_dev && a.pos - a.window + 1 > 0) ? a.pos - a.window + 1 : 0;
    long long n_keys = a.pos - lo_min + 1;
    if (a.window > 0 && n_keys > a.window) n_keys = a.window;
    const unsigned chunks = (unsigned)((n_keys + AT_CH - 1) / AT_CH);
    static bool configured = false;
    static int n_sms = 0;
    const int rep4 = (rep + 3) / 4;                       // the fused kernel keeps at most four heads per thread
    const size_t fused_smem = (size_t)rep * a.hd * 12 + (size_t)AT_CH * (a.hd + 4) * 4 + (size_t)AT_CH * a.hd * 4 + (size_t)AT_CH * AT_MAXREP * 4;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(attn_pv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(attn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return cudaGetLastError();
        int dev = 0, coop = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        if (!coop) n_sms = 0;
        configured = true;
    }
    // one CTA per SM where a KV head's keys, cut into n_sms / Hkv chunks, fit the shared memory of a CTA
    if (g_attn_fused == 1 && a.partial && n_sms > 0 && !a.batch && rep <= AF_HEADS && AF_THREADS % a.hd == 0 && a.hd % 32 == 0 &&
        a.fa <= 23 && a.Hkv <= 120) {                                       // probabilities (at most 2^fa) as three bytes
        static bool fat_configured = false;
        if (!fat_configured) {
            if (cudaFuncSetAttribute(attn_fat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024) != cudaSuccess) return cudaGetLastError();
            fat_configured = true;
        }
        const int per_head = std::max(1, std::min(n_sms, 192) / a.Hkv);      // the partial-sum scratch holds 192 chunks
        int C = (int)((n_keys + per_head - 1) / per_head);
        C = std::max(32, (C + 31) / 32 * 32);                      // whole 32-key steps of the tensor-core passes
        const unsigned fat_chunks = (unsigned)((n_keys + C - 1) / C);
        const size_t fat_smem = ((size_t)2 * C * a.hd + (size_t)C / 8 * 24) * 4 + (size_t)AF_HEADS * a.hd * 12 + (size_t)C * AF_HEADS * 4 +
                                (size_t)AF_THREADS / a.hd * AF_HEADS * a.hd * 8 + (size_t)4 * AF_HEADS * (a.hd + 16) + (size_t)3 * AF_HEADS * (C + 16);
        int per_sm = 0;
        if (C <= 2 * 8 * (AF_THREADS / 32) && fat_smem <= 208 * 1024 &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_fat_kernel, AF_THREADS, fat_smem) == cudaSuccess &&
            (long long)fat_chunks * a.Hkv <= (long long)per_sm * n_sms) {
            AttnArgs f = a;
            f.chunk = C;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(fat_chunks, a.Hkv); cfg.blockDim = dim3(AF_THREADS); cfg.dynamicSmemBytes = fat_smem; cfg.stream = s;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = a.pdl ? 2 : 1;
            const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_fat_kernel, f);
            note_launch(1);
            return e != cudaSuccess ? e : cudaGetLastError();
        }
        cudaGetLastError();
    }
    bool fused = g_attn_fused && a.partial && n_sms > 0 && rep4 <= 256 / AT_CH && fused_smem <= 200 * 1024;
    if (fused) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_fused_kernel, 256, fused_smem) != cudaSuccess) { cudaGetLastError(); per_sm = 0; }
        fused = (long long)chunks * a.Hkv <= (long long)per_sm * n_sms;      // a cooperative launch needs every CTA resident
    }
    if (fused) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(chunks, a.Hkv); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = fused_smem; cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = a.pdl ? 2 : 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_fused_kernel, a);
        note_launch(1);
        return e != cudaSuccess ? e : cudaGetLastError();
    }
    attn_scores_kernel<<<dim3(chunks, a.Hkv), 256, (size_t)rep * a.hd * 12 + (size_t)AT_CH * (a.hd + 4) * 4, s>>>(a);
    attn_exp_kernel<<<dim3((unsigned)((n_keys + 255) / 256), a.H), 256, 0, s>>>(a);
    attn_pv_kernel<<<dim3(chunks, a.Hkv), 256, (size_t)AT_CH * a.hd * 4 + (size_t)AT_CH * AT_MAXREP * 4, s>>>(a);
    note_launch(3);
    return cudaGetLastError();
}

cudaError_t launch_attn_prefill(const AttnArgs &a, cudaStream_t s) {
    const long long last_pos = a.seq_stride > 0 ? a.pos : a.pos + a.batch - 1;
    if (!attn_shape_ok(a.H, a.Hkv, a.hd) || a.batch <= 0 || a.batch > 65535 || a.pos < 0 || last_pos >= a.Lmax || a.seq_stride < 0 || a.fa < 1 ||
        a.fa > 29 || (a.rope && (!a.cos || !a.sin)) || a.pos_dev || !a.out || !a.scores || !a.e || !a.hmax || !a.Z)
        return cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(attn_pv_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
            return cudaGetLastError();
        configured = true;
    }
    const int rep = a.H / a.Hkv;
    const long long last = last_pos;                                // the longest key span is the last token's
    long long n_keys = last + 1;
    if (a.window > 0 && n_keys > a.window) n_keys = a.window;
    const unsigned chunks = (unsigned)((n_keys + AT_CH - 1) / AT_CH);
    attn_append_kernel<<<dim3((unsigned)a.batch, a.Hkv), 128, 0, s>>>(a);
    if (g_attn_fused != 0 && g_attn_tile_tc >= 0 && attn_tiles_ok(a)) {
        // consecutive tokens of one sequence: sixteen tokens per CTA share every staged chunk of keys and values
        note_launch(1);
        cudaError_t e = launch_attn_tile_scores(a, s);
        if (e == cudaSuccess) e = launch_attn_tile_exp(a, s);
        return e == cudaSuccess ? launch_attn_tile_pv(a, s) : e;
    }
    const bool tc = g_attn_fused != 0 && rep <= AF_HEADS && (a.hd == 64 || a.hd == 128);      // shapes the tensor-core kernel carries
    if (tc) {
        static bool tc_configured = false;
        if (!tc_configured) {
            if (cudaFuncSetAttribute(attn_scores_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
                return cudaGetLastError();
            tc_configured = true;
        }
        const size_t sc_smem = (size_t)AF_HEADS * a.hd * 8 + (size_t)2 * AT_CH * AF_HEADS * 8 + (size_t)2 * AT_CH * (a.hd + 4) * 4 +
                               (size_t)4 * AF_HEADS * (a.hd + 16);
        // longer walks amortise the query rotation and the pipeline start, as long as a few CTAs per SM remain
        AttnArgs t = a;
        const long long pairs = (long long)a.Hkv * a.batch;
        int walk = (int)((long long)chunks * pairs / (4 * 148));
        walk = walk < TS_CHUNKS_MIN ? TS_CHUNKS_MIN : walk > TS_CHUNKS_MAX ? TS_CHUNKS_MAX : walk;
        t.chunk = walk;
        attn_scores_tc_kernel<<<dim3((chunks + walk - 1) / walk, a.Hkv, (unsigned)a.batch), 256, sc_smem, s>>>(t);
    } else
        attn_scores_kernel<<<dim3(chunks, a.Hkv, (unsigned)a.batch), 256, (size_t)rep * a.hd * 12 + (size_t)AT_CH * (a.hd + 4) * 4, s>>>(a);
    attn_exp_kernel<<<dim3((unsigned)((n_keys + 255) / 256), a.H, (unsigned)a.batch), 256, 0, s>>>(a);
    const size_t pv_smem = (size_t)2 * AT_CH * a.hd * 4 + (size_t)AT_CH * AT_MAXREP * 4 + (size_t)(256 / a.hd) * 8 * a.hd * 8;
    if (256 % a.hd) return cudaErrorInvalidValue;                    // the probability x value pass splits 256 threads over the head dimension
    if (a.pv_splits > 1 && a.pv_part) {
        // few (token, KV head) pairs: the key chunks of a pair are shared out over pv_splits CTAs, a small launch adds their sums
        attn_pv_rows_kernel<<<dim3((unsigned)a.pv_splits, a.Hkv, (unsigned)a.batch), 256, pv_smem, s>>>(a);
        const long long n_out = (long long)a.batch * a.H * a.hd;
        attn_pv_finish_kernel<<<(unsigned)((n_out + 255) / 256), 256, 0, s>>>(a);
        note_launch(1);
    } else
        attn_pv_rows_kernel<<<dim3(1, a.Hkv, (unsigned)a.batch), 256, pv_smem, s>>>(a);
    note_launch(4);
    return cudaGetLastError();
}

cudaError_t launch_attn_reset(long long *hmax, unsigned long long *Z, long long *acc, unsigned *ticket, int H, int hd, cudaStream_t s) {
    attn_reset_kernel<<<1, 256, 0, s>>>(hmax, Z, acc, ticket, H, hd);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_embed_row(const uint8_t *w, int qtype, long long nb, const int *row_dev, long long row_host, int frac,
                             int64_t *out, cudaStream_t s) {
    embed_row_kernel<<<(unsigned)((nb * 256 + 255) / 256), 256, 0, s>>>(w, qtype, nb, row_dev, row_host, frac, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_embed_rows(const uint8_t *w, int qtype, long long nb, const int *rows_dev, int n_rows, int frac, int64_t *out, cudaStream_t s) {
    if (n_rows <= 0 || n_rows > 65535 || !rows_dev) return cudaErrorInvalidValue;
    embed_row_kernel<<<dim3((unsigned)((nb * 256 + 255) / 256), (unsigned)n_rows), 256, 0, s>>>(w, qtype, nb, rows_dev, 0, frac, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_argmax_rows(const int64_t *x, long long rows, long long n, int *out, cudaStream_t s) {
    if (n <= 0 || rows <= 0 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    argmax_rows_kernel<<<(unsigned)rows, 1024, 0, s>>>(x, n, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_argmax(const int64_t *x, long long n, int *out, cudaStream_t s) {
    if (n <= 0) return cudaErrorInvalidValue;
    long long ctas = (n + 8191) / 8192;
    argmax_kernel<<<(unsigned)(ctas > AM_CTAS ? AM_CTAS : ctas), 1024, 0, s>>>(x, n, out);
    note_launch();
    return cudaGetLastError();
}

}  // namespace iie
