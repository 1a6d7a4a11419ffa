// Support kernels around the streamed products: weight repack, activation limb planes, the exact
// 128-bit fallback product, routing (top-k + sigmoid), dispatch, RMSNorm and the unfused
// element-wise steps used by the fallback composition.
#include "kernels.h"
#include "layout.cuh"

namespace iie {

unsigned long long g_launches = 0;

namespace {

// ---------------------------------------------------------------------------------------------------
// repack / unpack: one thread per raw byte
// ---------------------------------------------------------------------------------------------------
template <bool FORWARD>
__global__ void repack_kernel(const uint8_t *src, uint8_t *dst, long long out_f, long long nb, int qtype,
                              unsigned *maxbits) {
    const int bs = qtype == QT_Q4K ? 144 : 210;
    const long long total = out_f * nb * bs;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long blk_lin = idx / bs;
        const int i = (int)(idx - blk_lin * bs);
        const long long row = blk_lin / nb, blk = blk_lin - row * nb;
        const long long unit = (row >> 3) * nb + blk;
        const int r = (int)(row & 7);
        const long long packed = qtype == QT_Q4K ? unit * HTB_Q4K + q4k_unit_offset(r, i)
                                                 : unit * HTB_Q6K + q6k_unit_offset(r, i);
        if (FORWARD) {
            dst[packed] = src[idx];
            if (maxbits) {                                  // block scale magnitudes (little-endian halves)
                const int dpos = qtype == QT_Q4K ? 0 : 208;
                if (i == dpos) atomicMax(&maxbits[0], ((unsigned)src[idx] | ((unsigned)src[idx + 1] << 8)) & 0x7FFFu);
                if (qtype == QT_Q4K && i == 2)
                    atomicMax(&maxbits[1], ((unsigned)src[idx] | ((unsigned)src[idx + 1] << 8)) & 0x7FFFu);
            }
        } else {
            dst[idx] = src[packed];
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// activation limb planes
// ---------------------------------------------------------------------------------------------------
__global__ void limbs_kernel(const int64_t *x, long long n_rows, long long K, int8_t *planes, int *flags, int *nl_out) {
    const long long total = n_rows * K;
    bool bad = false;
    int nl = 0;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / K, col = idx - row * K;
        bool ok;
        const uint64_t d = balanced_digits8(x[idx], ok);
        bad |= !ok;
        const int used = d == 0 ? 1 : 8 - (__clzll((long long)d) >> 3);
        nl = used > nl ? used : nl;
#pragma unroll
        for (int l = 0; l < 8; l++) planes[(row * 8 + l) * K + col] = (int8_t)(d >> (8 * l));
    }
    if (bad) atomicOr(flags, 1);
    if (nl_out && nl > 0) atomicMax(nl_out, nl);
}

// The same for K a multiple of 8: a thread takes eight consecutive columns (64 bytes in), transposes the 8 x 8 digit
// bytes in registers and writes eight bytes to each plane.
__global__ void __launch_bounds__(256) limbs8_kernel(const int64_t *__restrict__ x, long long n_rows, long long K, int8_t *__restrict__ planes,
                                                     int *flags, int *nl_out) {
    const long long per_row = K >> 3, total = n_rows * per_row;
    bool bad = false;
    uint64_t seen = 0;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
        const long long row = g / per_row, col = (g - row * per_row) << 3;
        const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(x + row * K + col);
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const ulonglong2 v = __ldg(src + i);
            bool ok0, ok1;
            const uint64_t d0 = balanced_digits8((int64_t)v.x, ok0), d1 = balanced_digits8((int64_t)v.y, ok1);
            bad |= !ok0 | !ok1;
            seen |= d0 | d1;                               // a digit position is in use if any element has a non-zero digit there or above
            lo[2 * i] = (uint32_t)d0; hi[2 * i] = (uint32_t)(d0 >> 32);
            lo[2 * i + 1] = (uint32_t)d1; hi[2 * i + 1] = (uint32_t)(d1 >> 32);
        }
        int8_t *dst = planes + row * 8 * K + col;
#pragma unroll
        for (int half = 0; half < 2; half++) {             // digits 0..3 from the low words, 4..7 from the high words
            const uint32_t *v = half ? hi : lo;
            uint32_t a[4], b[4];                           // a: elements 0..3, b: elements 4..7, one word per digit
            {
                const uint32_t t0 = __byte_perm(v[0], v[1], 0x5140), t1 = __byte_perm(v[2], v[3], 0x5140);
                const uint32_t t2 = __byte_perm(v[0], v[1], 0x7362), t3 = __byte_perm(v[2], v[3], 0x7362);
                a[0] = __byte_perm(t0, t1, 0x5410); a[1] = __byte_perm(t0, t1, 0x7632);
                a[2] = __byte_perm(t2, t3, 0x5410); a[3] = __byte_perm(t2, t3, 0x7632);
            }
            {
                const uint32_t t0 = __byte_perm(v[4], v[5], 0x5140), t1 = __byte_perm(v[6], v[7], 0x5140);
                const uint32_t t2 = __byte_perm(v[4], v[5], 0x7362), t3 = __byte_perm(v[6], v[7], 0x7362);
                b[0] = __byte_perm(t0, t1, 0x5410); b[1] = __byte_perm(t0, t1, 0x7632);
                b[2] = __byte_perm(t2, t3, 0x5410); b[3] = __byte_perm(t2, t3, 0x7632);
            }
#pragma unroll
            for (int l = 0; l < 4; l++) *reinterpret_cast<uint2 *>(dst + (half * 4 + l) * K) = make_uint2(a[l], b[l]);
        }
    }
    if (bad) atomicOr(flags, 1);
    if (nl_out) {
        // digits in use = position of the highest non-zero digit byte over all elements seen (at least one)
        const int nl = seen == 0 ? 1 : 8 - (__clzll((long long)seen) >> 3);
        atomicMax(nl_out, nl);
    }
}

// ---------------------------------------------------------------------------------------------------
// exact fallback: one thread per output, 128-bit accumulation in the reference's per-weight form
// (north-mini-code/tools/nmc_qk_kernel.c:85-120).  Valid for every int64 input.
// ---------------------------------------------------------------------------------------------------
__global__ void exact_linear_kernel(const uint8_t *w, int qtype, long long out_f, long long nb, const int64_t *x,
                                    long long T, int fw, int64_t *out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= out_f * T) return;
    const long long o = idx % out_f, t = idx / out_f;
    const int64_t *xt = x + t * nb * 256;
    i128 acc = 0;
    for (long long b = 0; b < nb; b++) {
        const int64_t *xb = xt + b * 256;
        auto byte = [&](int i) { return (int)repacked_byte(w, qtype, nb, o, b, i); };
        if (qtype == QT_Q4K) {
            const int64_t dq = half_to_fixed(byte(0) | (byte(1) << 8), fw), dmq = half_to_fixed(byte(2) | (byte(3) << 8), fw);
            for (int j = 0; j < 8; j++) {
                int sc, mn;
                if (j < 4) { sc = byte(4 + j) & 63; mn = byte(8 + j) & 63; }
                else { sc = (byte(8 + j) & 0xF) | ((byte(j) >> 6) << 4); mn = (byte(8 + j) >> 4) | ((byte(4 + j) >> 6) << 4); }
                const int64_t ws = dq * sc, wm = dmq * mn;
                for (int l = 0; l < 32; l++) {
                    const int q = (byte(16 + 32 * (j >> 1) + l) >> ((j & 1) * 4)) & 0xF;
                    acc += (i128)(ws * q - wm) * xb[32 * j + l];
                }
            }
        } else {
            const int64_t dq = half_to_fixed(byte(208) | (byte(209) << 8), fw);
            for (int sb = 0; sb < 16; sb++) {
                const int half = sb >> 3, k = (sb >> 1) & 3, l0 = (sb & 1) * 16;
                const int64_t ws = dq * (int64_t)(int8_t)byte(192 + 8 * half + 2 * k + (sb & 1));
                for (int l = 0; l < 16; l++) {
                    const int ql = byte(64 * half + 32 * (k & 1) + l0 + l), qh = byte(128 + 32 * half + l0 + l);
                    const int q = (((k < 2) ? (ql & 0xF) : (ql >> 4)) | (((qh >> (2 * k)) & 3) << 4)) - 32;
                    acc += (i128)(ws * q) * xb[16 * sb + l];
                }
            }
        }
    }
    out[t * out_f + o] = (int64_t)(acc >> fw);
}

// Dense int64 weights (router / gain matrices registered as int64): exact 128-bit product; the
// reference additionally requires the un-shifted sum to fit int64 (nmc_qk_cuda.cu:615-638), which is
// reported through flags bit 2.
__global__ void exact_dense_kernel(const int64_t *w, long long out_f, long long in_f, const int64_t *x, long long T,
                                   int fw, int64_t *out, int *flags) {
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= out_f * T) return;
    const long long o = warp % out_f, t = warp / out_f;
    i128 acc = 0;
    for (long long i = lane; i < in_f; i += 32) acc += (i128)w[o * in_f + i] * x[t * in_f + i];
    unsigned long long lo = (unsigned long long)acc, hi = (unsigned long long)((u128)acc >> 64);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const unsigned long long lo2 = __shfl_down_sync(0xffffffffu, lo, s), hi2 = __shfl_down_sync(0xffffffffu, hi, s);
        const u128 sum = (((u128)hi << 64) | lo) + (((u128)hi2 << 64) | lo2);
        lo = (unsigned long long)sum; hi = (unsigned long long)(sum >> 64);
    }
    if (lane == 0) {
        const i128 total = (i128)(((u128)hi << 64) | lo);
        if (total > (i128)INT64_MAX || total < (i128)INT64_MIN) { if (flags) atomicOr(flags, 4); out[t * out_f + o] = 0; }
        else out[t * out_f + o] = ((int64_t)total) >> fw;
    }
}

__global__ void silu_mul_kernel(int64_t *a, const int64_t *b, long long n, int fa) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = mul_shift(silu_fixed(a[i], fa), b[i], fa);
}

__global__ void combine_kernel(const int64_t *dn, const int64_t *gates, long long T, int k, long long d_model, int fa,
                               int64_t *out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * d_model) return;
    const long long t = i / d_model, o = i - t * d_model;
    unsigned long long acc = 0;
    for (int j = 0; j < k; j++) acc += (unsigned long long)mul_shift(dn[(t * k + j) * d_model + o], gates[t * k + j], fa);
    out[i] = (int64_t)acc;
}

// ---------------------------------------------------------------------------------------------------
// top-k with lowest-index tie-break + sigmoid gates (north-mini-code/src/nmc/cohere2.py:162-165,180)
// ---------------------------------------------------------------------------------------------------
__global__ void topk_kernel(const int64_t *logits, long long rows, int n_experts, int k, int fa, int *ids,
                            int64_t *gates) {
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int64_t *lr = logits + row * n_experts;
    unsigned taken = 0;                                   // bit i: element lane + 32*i already selected
    for (int r = 0; r < k; r++) {
        int64_t best = INT64_MIN; int best_id = 0x7fffffff;
        for (int i = 0, e = lane; e < n_experts; i++, e += 32) {
            if (taken & (1u << i)) continue;
            const int64_t v = lr[e];
            if (best_id == 0x7fffffff || v > best) { best = v; best_id = e; }   // ascending e: ties keep the lower id
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const int64_t ov = __shfl_xor_sync(0xffffffffu, best, s);
            const int oi = __shfl_xor_sync(0xffffffffu, best_id, s);
            if (oi != 0x7fffffff && (best_id == 0x7fffffff || ov > best || (ov == best && oi < best_id))) { best = ov; best_id = oi; }
        }
        if (best_id != 0x7fffffff && (best_id & 31) == lane) taken |= 1u << (best_id >> 5);
        if (lane == 0) {
            ids[row * k + r] = best_id == 0x7fffffff ? -1 : best_id;
            gates[row * k + r] = best_id == 0x7fffffff ? 0 : sigmoid_fixed(best, fa);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// dispatch: stable counting sort of (token, slot) pairs by expert, single CTA.  Warp w owns the w-th
// contiguous slice of the pair list; inside a slice, 32 pairs at a time are ranked with a warp match,
// so expert e's pairs keep ascending pair index.  Slots whose expert id falls outside
// [expert_base, expert_base + n_experts) are dropped (they belong to another expert shard).
// ---------------------------------------------------------------------------------------------------
__global__ void dispatch_kernel(const int *ids, const int64_t *gates, long long T, int k, int n_experts, int expert_base,
                                int *grp_off, int *pair_tok, int64_t *pair_gate) {
    extern __shared__ int sm[];                           // cnt[nwarps][E], then start[E + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int *cnt = sm, *start = sm + nwarps * n_experts;
    const long long P = T * k;
    const long long per = ((P + nwarps - 1) / nwarps + 31) / 32 * 32;      // slice length, a multiple of 32
    const long long lo = (long long)warp * per, hi = lo + per < P ? lo + per : P;
    for (int i = threadIdx.x; i < nwarps * n_experts; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    int *mine = cnt + warp * n_experts;
    for (long long i0 = lo; i0 < hi; i0 += 32) {
        const long long i = i0 + lane;
        int e = i < hi ? ids[i] - expert_base : -1;
        if (e < 0 || e >= n_experts) e = -1;
        const unsigned m = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(m) - 1) mine[e] += __popc(m);
        __syncwarp();
    }
    __syncthreads();
    // per expert: slice counts -> slice offsets inside the expert's range; then the ranges themselves
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        int run = 0;
        for (int w = 0; w < nwarps; w++) { const int c = cnt[w * n_experts + e]; cnt[w * n_experts + e] = run; run += c; }
        start[e] = run;                                  // total of expert e for now
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; e++) { const int c = start[e]; start[e] = run; grp_off[e] = run; run += c; }
        start[n_experts] = run; grp_off[n_experts] = run;
    }
    __syncthreads();
    for (long long i0 = lo; i0 < hi; i0 += 32) {
        const long long i = i0 + lane;
        int e = i < hi ? ids[i] - expert_base : -1;
        if (e < 0 || e >= n_experts) e = -1;
        const unsigned m = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int dst = start[e] + mine[e] + __popc(m & ((1u << lane) - 1));
            pair_tok[dst] = (int)(i / k);
            pair_gate[dst] = gates[i];
        }
        __syncwarp();
        if (e >= 0 && lane == __ffs(m) - 1) mine[e] += __popc(m);
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------------
// integer RMSNorm (north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72), one CTA per row
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long uabs64(int64_t v) { return v < 0 ? (0ULL - (unsigned long long)v) : (unsigned long long)v; }

__device__ u128 isqrt_u128(u128 v) {
    u128 res = 0, bit = (u128)1 << 126;
    while (bit > v) bit >>= 2;
    while (bit != 0) {
        if (v >= res + bit) { v -= res + bit; res = (res >> 1) + bit; } else res >>= 1;
        bit >>= 2;
    }
    return res;
}

// floor(sqrt(v)): a double estimate fixed up with exact 128-bit products while v < 2^104, else the bitwise root
__device__ u128 isqrt_fast(u128 v) {
    if (v < ((u128)1 << 104)) {
        const double dv = (double)(unsigned long long)(v >> 64) * 18446744073709551616.0 + (double)(unsigned long long)v;
        unsigned long long r = (unsigned long long)sqrt(dv);
        for (int it = 0; it < 8 && (u128)r * r > v; it++) r--;
        for (int it = 0; it < 8 && (u128)(r + 1) * (r + 1) <= v; it++) r++;
        if ((u128)r * r <= v && (u128)(r + 1) * (r + 1) > v) return r;
    }
    return isqrt_u128(v);
}

// one element of the normalised row: floor((x << fa) / rms), then (y * gain) >> fa; `bad` is set (and 0 returned)
// where the oracle's envelope checks would refuse the value
__device__ __forceinline__ int64_t norm_value(int64_t xv, unsigned long long rms, unsigned long long inv, unsigned long long gm,
                                              int64_t g, bool has_gain, int fa, bool &bad) {
    int64_t y;
    if (inv != 0 && uabs64(xv) < (1ULL << (62 - fa))) {
        // |x << fa| < 2^62 and rms < 2^62: quotient from the reciprocal inv = floor((2^64 - 1) / rms), at most 2 low
        const unsigned long long n = uabs64(xv) << fa;
        unsigned long long q = __umul64hi(n, inv), r = n - q * rms;
        while (r >= rms) { q++; r -= rms; }
        y = xv >= 0 ? (int64_t)q : -(int64_t)q - (r != 0);      // floor toward -inf
    } else {
        const i128 num = (i128)xv << fa;
        i128 q = num / (i128)rms;
        if (num < 0 && q * (i128)rms != num) q -= 1;
        if (q > (i128)INT64_MAX || q < (i128)INT64_MIN) { bad = true; return 0; }
        y = (int64_t)q;
    }
    if (has_gain) {
        // the oracle refuses a gain product that could leave int64
        if ((u128)uabs64(y) * gm > (u128)INT64_MAX) { bad = true; return 0; }
        y = (int64_t)(((i128)y * g) >> fa);
    }
    return y;
}

// rows from `rows_a` on use gain_b (per-head norms of queries and keys in one launch)
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const int64_t *x, long long rows, long long width, const int64_t *gain_a,
                                                       int fa, unsigned long long eps, int64_t *out, int *flags,
                                                       int8_t *planes, int64_t *totals, const int64_t *gain_b, long long rows_a,
                                                       int split) {
    // `split` CTAs share a row: each sums the squares of the whole row (cheap, the row sits in L2) and normalises its own
    // slice, so that the divisions of a long row are spread over several SMs
    __shared__ unsigned long long s_lo[32], s_hi[32], s_max[32], s_gmax[32];
    __shared__ unsigned long long s_rms, s_gm, s_inv;
    __shared__ int s_bad;
    const long long row = blockIdx.x / split;
    const int part = blockIdx.x - (int)row * split;
    const int64_t *gain = row < rows_a ? gain_a : gain_b;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int64_t *xr = x + row * width;
    int64_t *yr = out + row * width;
    u128 ssq = 0; unsigned long long mx = 0, gmx = 0;
    for (long long i0 = tid; i0 < width; i0 += (long long)blockDim.x * 8) {      // eight loads in flight per thread
        int64_t xv[8], gv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const long long i = i0 + (long long)u * blockDim.x;
            xv[u] = i < width ? xr[i] : 0;
            gv[u] = (gain && i < width) ? gain[i] : 0;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const unsigned long long a = uabs64(xv[u]), ga = uabs64(gv[u]);
            ssq += (u128)a * a;
            mx = a > mx ? a : mx;
            gmx = ga > gmx ? ga : gmx;
        }
    }
    auto fold = [&]() {
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const unsigned long long lo = __shfl_down_sync(0xffffffffu, (unsigned long long)ssq, off);
            const unsigned long long hi = __shfl_down_sync(0xffffffffu, (unsigned long long)(ssq >> 64), off);
            const unsigned long long m2 = __shfl_down_sync(0xffffffffu, mx, off), g2 = __shfl_down_sync(0xffffffffu, gmx, off);
            ssq += ((u128)hi << 64) | lo;
            mx = m2 > mx ? m2 : mx; gmx = g2 > gmx ? g2 : gmx;
        }
    };
    fold();
    if (lane == 0) { s_lo[warp] = (unsigned long long)ssq; s_hi[warp] = (unsigned long long)(ssq >> 64); s_max[warp] = mx; s_gmax[warp] = gmx; }
    __syncthreads();
    if (warp == 0) {
        ssq = lane < nwarps ? (((u128)s_hi[lane] << 64) | s_lo[lane]) : (u128)0;
        mx = lane < nwarps ? s_max[lane] : 0; gmx = lane < nwarps ? s_gmax[lane] : 0;
        fold();
        if (lane == 0) {
            // |x| <= 2^57 keeps the 128-bit sum of squares exact for any width <= 2^13
            int bad = (mx > (1ULL << 57) || width > 8192) ? 1 : 0;
            const u128 mean = ((width & (width - 1)) == 0 ? ssq >> (63 - __clzll(width)) : ssq / (u128)(unsigned long long)width) + eps;
            const u128 rms = isqrt_fast(mean);
            if (rms == 0 || rms > (u128)0xFFFFFFFFFFFFFFFFULL) bad = 1;
            s_rms = (unsigned long long)rms; s_gm = gmx; s_bad = bad;
            s_inv = (rms != 0 && rms < ((u128)1 << 62)) ? 0xFFFFFFFFFFFFFFFFULL / (unsigned long long)rms : 0ULL;
        }
    }
    __syncthreads();
    if (s_bad) { if (tid == 0 && part == 0) atomicOr(flags, 2); return; }
    const unsigned long long rms = s_rms, inv = s_inv;
    const unsigned long long gm = s_gm;
    bool bad = false;
    if (planes) {
        // digit planes [row][8][width] and 128-element block sums of the normalised row, for the Q1_0 product
        const long long nb = width >> 7, per = (nb + split - 1) / split;
        const long long b_end = min(nb, (part + 1) * per);
        for (long long b = part * per + warp; b < b_end; b += nwarps) {
            const long long i0 = b * 128 + lane * 4;
            uint32_t pl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            unsigned long long sum = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int64_t y = norm_value(xr[i0 + j], rms, inv, gm, gain ? gain[i0 + j] : 0, gain != nullptr, fa, bad);
                if (out) yr[i0 + j] = y;
                bool ok;
                const uint64_t d = balanced_digits8(y, ok);
                sum += (unsigned long long)y;
#pragma unroll
                for (int l = 0; l < 8; l++) pl[l] |= (uint32_t)((d >> (8 * l)) & 0xFF) << (8 * j);
            }
#pragma unroll
            for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + (row * 8 + l) * width + i0) = pl[l];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (lane == 0) totals[row * nb + b] = (int64_t)sum;
        }
    } else {
        const long long per = (width + split - 1) / split, i_end = min(width, (part + 1) * per);
        for (long long i = part * per + tid; i < i_end; i += blockDim.x)
            yr[i] = norm_value(xr[i], rms, inv, gm, gain ? gain[i] : 0, gain != nullptr, fa, bad);
    }
    if (bad) atomicOr(flags, 2);
}

inline unsigned grid_for(long long n, int tpb, long long cap = 148LL * 64) {
    long long g = (n + tpb - 1) / tpb;
    if (g > cap) g = cap;
    return (unsigned)(g < 1 ? 1 : g);
}

}  // namespace

cudaError_t launch_repack(const uint8_t *raw, uint8_t *dst, long long out_f, long long nb, int qtype,
                          unsigned *maxbits, cudaStream_t s) {
    const long long total = out_f * nb * (qtype == QT_Q4K ? 144 : 210);
    repack_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(raw, dst, out_f, nb, qtype, maxbits);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_unpack(const uint8_t *src, uint8_t *raw, long long out_f, long long nb, int qtype, cudaStream_t s) {
    const long long total = out_f * nb * (qtype == QT_Q4K ? 144 : 210);
    repack_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(src, raw, out_f, nb, qtype, nullptr);
    note_launch();
    return cudaGetLastError();
}

__global__ void set2_kernel(int *p, int a, int b) { p[0] = a; p[1] = b; }

cudaError_t launch_set2(int *p, int a, int b, cudaStream_t s) {
    set2_kernel<<<1, 1, 0, s>>>(p, a, b);
    note_launch();
    return cudaGetLastError();
}

// Selected experts without a binding, compacted in routing order: cold[0] = how many, cold[1..] = their ids
// (north-mini-code/tools/nmc_qk_cuda.cu cold_routes_k).  An id outside the table raises flag bit 1.
__global__ void cold_routes_kernel(const int *ids, int k, const unsigned char *bound, int n_experts, int *cold, int *flags) {
    int n = 0;
    for (int i = 0; i < k; i++) {
        const int e = ids[i];
        if (e < 0 || e >= n_experts) { atomicOr(flags, 2); continue; }
        if (!bound[e]) cold[1 + n++] = e;
    }
    cold[0] = n;
}

cudaError_t launch_cold_routes(const int *ids, int k, const unsigned char *bound, int n_experts, int *cold, int *flags, cudaStream_t s) {
    cold_routes_kernel<<<1, 1, 0, s>>>(ids, k, bound, n_experts, cold, flags);
    note_launch();
    return cudaGetLastError();
}

__global__ void add_rows_kernel(const int64_t *a, const int64_t *b, int64_t *out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (int64_t)((uint64_t)a[i] + (uint64_t)b[i]);
}

cudaError_t launch_add_rows(const int64_t *a, const int64_t *b, int64_t *out, long long n, cudaStream_t s) {
    add_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, out, n);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_limbs(const int64_t *x, long long n_rows, long long K, int8_t *planes, int *flags, cudaStream_t s,
                         int *nl_out) {
    if (K % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(planes) & 7) == 0)
        limbs8_kernel<<<grid_for(n_rows * (K >> 3), 256), 256, 0, s>>>(x, n_rows, K, planes, flags, nl_out);
    else
        limbs_kernel<<<grid_for(n_rows * K, 256), 256, 0, s>>>(x, n_rows, K, planes, flags, nl_out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_exact_linear(const uint8_t *w, int qtype, long long out_f, long long nb, const int64_t *x,
                                long long T, int fw, int64_t *out, cudaStream_t s) {
    const long long n = out_f * T;
    exact_linear_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(w, qtype, out_f, nb, x, T, fw, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_exact_dense(const int64_t *w, long long out_f, long long in_f, const int64_t *x, long long T,
                               int fw, int64_t *out, int *flags, cudaStream_t s) {
    const long long n = out_f * T * 32;
    exact_dense_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(w, out_f, in_f, x, T, fw, out, flags);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(int64_t *a, const int64_t *b, long long n, int fa, cudaStream_t s) {
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, n, fa);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_combine(const int64_t *dn, const int64_t *gates, long long T, int k, long long d_model, int fa,
                           int64_t *out, cudaStream_t s) {
    const long long n = T * d_model;
    combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(dn, gates, T, k, d_model, fa, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_topk(const int64_t *logits, long long rows, int n_experts, int k, int fa, int *ids, int64_t *gates,
                        cudaStream_t s) {
    if (n_experts > 1024 || n_experts <= 0 || k <= 0) return cudaErrorInvalidValue;
    const long long n = rows * 32;
    topk_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(logits, rows, n_experts, k, fa, ids, gates);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm(const int64_t *x, long long rows, long long width, const int64_t *gain, int fa,
                           unsigned long long eps, int64_t *out, int *flags, cudaStream_t s) {
    const int split = (rows <= 16 && width >= 1024) ? (int)((width + 511) / 512) : 1;      // few long rows: 512 values per CTA
    const int threads = split > 1 ? 128 : (width >= 2048 ? 1024 : width > 128 ? 256 : 128);
    rmsnorm_kernel<<<(unsigned)(rows * split), threads, 0, s>>>(x, rows, width, gain, fa, eps, out, flags, nullptr, nullptr, nullptr, rows,
                                                                 split);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm_pair(const int64_t *x, long long rows_a, long long rows_b, long long width, const int64_t *gain_a,
                                const int64_t *gain_b, int fa, unsigned long long eps, int64_t *out, int *flags, cudaStream_t s) {
    const int threads = width >= 2048 ? 1024 : width > 128 ? 256 : 128;
    rmsnorm_kernel<<<(unsigned)(rows_a + rows_b), threads, 0, s>>>(x, rows_a + rows_b, width, gain_a, fa, eps, out, flags, nullptr, nullptr,
                                                                  gain_b, rows_a, 1);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm_planes(const int64_t *x, long long rows, long long width, const int64_t *gain, int fa,
                                  unsigned long long eps, int64_t *out, int8_t *planes, int64_t *totals, int *flags, cudaStream_t s) {
    if (width <= 0 || (width & 127) || !planes || !totals) return cudaErrorInvalidValue;
    // one warp per 128-element block; few rows of a long row: four blocks per CTA, several CTAs per row
    const long long nb = width >> 7;
    const int split = (rows <= 16 && nb >= 8) ? (int)((nb + 3) / 4) : 1;
    const int threads = split > 1 ? 128 : (width >= 4096 ? 1024 : width >= 1024 ? (int)(width >> 2) : 256);
    rmsnorm_kernel<<<(unsigned)(rows * split), threads, 0, s>>>(x, rows, width, gain, fa, eps, out, flags, planes, totals, nullptr, rows,
                                                                 split);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_dispatch(const int *ids, const int64_t *gates, long long T, int k, int n_experts, int *grp_off,
                            int *pair_tok, int64_t *pair_gate, cudaStream_t s, int expert_base) {
    if (n_experts > 1024 || n_experts <= 0) return cudaErrorInvalidValue;
    const int warps = n_experts <= 320 ? 32 : 8;                        // cnt[warps][E] + start[E + 1] stays below 48 KB
    const size_t smem = ((size_t)warps * n_experts + n_experts + 1) * sizeof(int);
    dispatch_kernel<<<1, 32 * warps, smem, s>>>(ids, gates, T, k, n_experts, expert_base, grp_off, pair_tok, pair_gate);
    note_launch();
    return cudaGetLastError();
}

}  // namespace iie
