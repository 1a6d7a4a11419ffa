// Q1_0 (one sign bit per weight, one integer scale per 128-weight block) linear products.
//
// Contract (bonsai/src/trinote/infer_int/reference_bonsai.py:149-219, bonsai/tools/bonsai_q1_kernel.c:85-106,
// bonsai/tools/bonsai_q1_gpu.cu:78-123):
//     out[t,o] = sum_b arshift( (sum_{i<128} s_i x[t,128b+i]) * scale[o,b]  mod 2^64, frac )        (mod 2^64)
// with s_i = +1 for a set bit (little-endian inside each byte) and -1 for a clear one, the shift flooring
// toward minus infinity and applied per block BEFORE the blocks are added.
//
// The reference spends one warp on every (token, row) output and adds 128 int64 values per block on the
// CUDA cores.  Here the block sums run on the tensor cores and stay exact modulo 2^64:
//   * sum_i s_i x_i = 2 * P - S with P = sum over set bits of x_i and S = sum_i x_i; S does not depend on
//     the weight row and is formed once per (token, block) while the activations are split into digits;
//   * x = sum_l 256^l d_l (mod 2^64) with eight balanced digits d_l in [-128,127] (the carry out of the
//     eighth digit is a multiple of 2^64 and drops out), so P = sum_l 256^l sum_i bit_i d_{l,i} (mod 2^64):
//     the eight digit planes are the N = 8 columns of an int8 warp MMA whose A operand is the weight
//     bits expanded to bytes 0/1.  |sum_i bit_i d_{l,i}| <= 128*128, far inside int32.  Every int64 input
//     is therefore handled exactly; there is no envelope and no fallback.
//
// Weight layout ("units"): rows are grouped in tiles of 16; unit (tile, block) holds 256 bytes of sign
// bits in MMA A-fragment order followed by the 16 block scales (int32 when every scale of the matrix
// fits, else int64).  Lane (g,t) owns two 32-bit words; bit r + 8 i of word mp is the sign bit of row
// g + 8 (r & 1), column 32 (2 mp + (r >> 2)) + 8 t + 4 ((r >> 1) & 1) + i, so A register j of MMA m is
// (word[m >> 1] >> (4 (m & 1) + j)) & 0x01010101: two instructions per register.
#include "kernels.h"
#include "mma_items.cuh"

namespace iie {

namespace {

__device__ __forceinline__ int64_t q1_shift(int64_t v, int sh) { return v >> sh; }   // arithmetic: floors

// ---- registration: raw [out_f][nb][16] bits + [out_f][nb] scales -> units ------------------------------------
template <typename ST, typename DT>
__global__ void q1_repack_kernel(const uint8_t *bits, const ST *scale, long long out_f, long long nb, long long n_tiles,
                                 uint8_t *units) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;     // (tile, block, slot 0..79)
    const long long n = n_tiles * nb * 80;
    if (idx >= n) return;
    const int slot = (int)(idx % 80);
    const long long tb = idx / 80, tile = tb / nb, b = tb - tile * nb;
    uint8_t *unit = units + tb * US;
    if (slot < 64) {
        const int lane = slot >> 1, mp = slot & 1, g = lane >> 2, t = lane & 3;
        uint32_t w = 0;
        for (int p = 0; p < 32; p++) {
            const int r = p & 7, i = p >> 3;
            const long long row = tile * 16 + g + 8 * (r & 1);
            const int k = 32 * (2 * mp + (r >> 2)) + 8 * t + 4 * ((r >> 1) & 1) + i;
            if (row < out_f) w |= (uint32_t)((bits[(row * nb + b) * 16 + (k >> 3)] >> (k & 7)) & 1) << p;
        }
        reinterpret_cast<uint32_t *>(unit)[lane * 2 + mp] = w;
    } else {
        const int r = slot - 64;
        const long long row = tile * 16 + r;
        reinterpret_cast<DT *>(unit + 256)[r] = row < out_f ? (DT)scale[row * nb + b] : (DT)0;
    }
}

// ---- activations: digit planes [tok][8][K], block sums [tok][nb], digits in use ---------------------------
// With `up` the activation is the SwiGLU of two rows of width K: ((x * sigmoid(x)) >> frac) * up >> frac, wrapping products;
// x and up then advance by `ld` per token.
__global__ void q1_prep_kernel(const int64_t *x, const int64_t *up, long long ld, int frac, int64_t log2e, int64_t clip, long long T,
                               long long nb, int8_t *planes, int64_t *totals, int *nl_out) {
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= T * nb) return;
    const long long tok = wid / nb, b = wid - tok * nb, K = nb * 128;
    const int64_t *src = x + tok * (up ? ld : K) + b * 128 + lane * 4;
    const longlong2 v0 = *reinterpret_cast<const longlong2 *>(src), v1 = *reinterpret_cast<const longlong2 *>(src + 2);
    int64_t v[4] = {v0.x, v0.y, v1.x, v1.y};
    if (up) {
        const int64_t *us = up + tok * ld + b * 128 + lane * 4;
        const longlong2 u0 = *reinterpret_cast<const longlong2 *>(us), u1 = *reinterpret_cast<const longlong2 *>(us + 2);
        const int64_t u[4] = {u0.x, u0.y, u1.x, u1.y};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t sg = sigmoid_fixed_c(v[i], frac, log2e, clip);
            const int64_t silu = (int64_t)((unsigned long long)v[i] * (unsigned long long)sg) >> frac;
            v[i] = (int64_t)((unsigned long long)silu * (unsigned long long)u[i]) >> frac;
        }
    }
    uint32_t pl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    unsigned long long sum = 0;
    int nl = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        bool ok;
        const uint64_t d = balanced_digits8(v[i], ok);
        nl = max(nl, ok ? digits_used(d) : 9);
        sum += (unsigned long long)v[i];
#pragma unroll
        for (int l = 0; l < 8; l++) pl[l] |= (uint32_t)((d >> (8 * l)) & 0xFF) << (8 * i);
    }
#pragma unroll
    for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + (tok * 8 + l) * K + b * 128 + lane * 4) = pl[l];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, off));
    }
    if (lane == 0) {
        totals[tok * nb + b] = (int64_t)sum;
        if (nl_out) atomicMax(nl_out, nl);
    }
}

struct Q1Args {
    const uint8_t *units;
    long long out_f, nb, n_tiles, T;
    int sh;                         // floor shift, already clamped to 0..63
    int tiles_per_cta;
    const int8_t *xl;               // [T][8][K]
    const int64_t *totals;          // [T][nb]
    int64_t *out;                   // [T][out_f]
    const int64_t *add;             // optional [T][out_f] added to the product (may be `out` itself)
    int *flags;                     // optional: bit 3 is raised when a bulk copy never arrived
};

// A fragments of MMA m from the two bit words of a lane
__device__ __forceinline__ void q1_afrag(const uint2 w, int m, uint32_t (&a)[4]) {
    const uint32_t word = (m >> 1) ? w.y : w.x;
    const int base = 4 * (m & 1);
#pragma unroll
    for (int j = 0; j < 4; j++) a[j] = (word >> (base + j)) & 0x01010101u;
}

// this lane's share of P for the two rows it sees: columns 2t, 2t+1 carry digits t and t+4
__device__ __forceinline__ void q1_partials(const int (&c)[4], int t, unsigned long long &lo, unsigned long long &hi) {
    lo = ((unsigned long long)(long long)c[0] << (8 * t)) + ((unsigned long long)(long long)c[1] << (8 * t + 32));
    hi = ((unsigned long long)(long long)c[2] << (8 * t)) + ((unsigned long long)(long long)c[3] << (8 * t + 32));
}

template <typename DT>
__device__ __forceinline__ int64_t q1_scale_at(const uint8_t *unit, int row) {
    return (int64_t)__ldg(reinterpret_cast<const DT *>(unit + 256) + row);
}

// ---- single token: warps split K, the activation fragments stay in registers, the CTA walks tiles -----
template <int BPW, typename DT>
__global__ void __launch_bounds__(512) q1_gemv_kernel(const Q1Args a) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    extern __shared__ unsigned long long q1_red[];                 // [tiles_per_cta][16]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long long K = a.nb * 128;
    const long long tile0 = (long long)blockIdx.x * a.tiles_per_cta;
    const int ntile = (int)min((long long)a.tiles_per_cta, a.n_tiles - tile0);
    for (int i = threadIdx.x; i < a.tiles_per_cta * 16; i += blockDim.x) q1_red[i] = 0ULL;
    __syncthreads();

    uint32_t bf[BPW][8];
    unsigned long long tot[BPW];
    const int8_t *xcol = a.xl + (long long)col_limb(g) * K + 8 * t;
#pragma unroll
    for (int i = 0; i < BPW; i++) {
        const long long b = warp + (long long)i * W;
        tot[i] = 0;
#pragma unroll
        for (int m = 0; m < 4; m++) { bf[i][2 * m] = 0; bf[i][2 * m + 1] = 0; }
        if (b < a.nb) {
            tot[i] = (unsigned long long)__ldg(a.totals + b);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint2 v = ldg64(xcol + b * 128 + 32 * m);
                bf[i][2 * m] = v.x; bf[i][2 * m + 1] = v.y;
            }
        }
    }

    const int myrow = g + 8 * (t & 1);
    // the bits and scales of the next tile are requested before the current one is multiplied
    uint2 wn[BPW];
    DT scn[BPW];
    auto fetch = [&](int tl) {
        const uint8_t *tile_units = a.units + (tile0 + tl) * a.nb * US;
#pragma unroll
        for (int i = 0; i < BPW; i++) {
            const long long b = warp + (long long)i * W;
            wn[i] = make_uint2(0, 0); scn[i] = 0;
            if (b < a.nb && tl < ntile) {
                const uint8_t *unit = tile_units + b * US;
                wn[i] = ldg64(unit + lane * 8);
                scn[i] = __ldg(reinterpret_cast<const DT *>(unit + 256) + myrow);
            }
        }
    };
    fetch(0);
    for (int tl = 0; tl < ntile; tl++) {
        uint2 w[BPW];
        int64_t sc[BPW];
#pragma unroll
        for (int i = 0; i < BPW; i++) { w[i] = wn[i]; sc[i] = (int64_t)scn[i]; }
        fetch(tl + 1);
        unsigned long long acc = 0;
#pragma unroll
        for (int i = 0; i < BPW; i++) {
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                uint32_t af[4];
                q1_afrag(w[i], m, af);
                mma_u8s8_k32(c, af[0], af[1], af[2], af[3], bf[i][2 * m], bf[i][2 * m + 1]);
            }
            unsigned long long lo, hi;
            q1_partials(c, t, lo, hi);
            // reduce-scatter over the four lanes of a row group: even t ends with row g, odd t with row g + 8
            const unsigned long long send = (t & 1) ? lo : hi;
            unsigned long long mine = ((t & 1) ? hi : lo) + __shfl_xor_sync(0xffffffffu, send, 1);
            mine += __shfl_xor_sync(0xffffffffu, mine, 2);
            const unsigned long long s = 2ULL * mine - tot[i];
            acc += (unsigned long long)q1_shift((int64_t)(s * (unsigned long long)sc[i]), a.sh);
        }
        if (t < 2) atomicAdd(&q1_red[tl * 16 + myrow], acc);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ntile * 16; i += blockDim.x) {
        const long long row = tile0 * 16 + i;
        if (row < a.out_f) a.out[row] = (int64_t)(q1_red[i] + (a.add ? (unsigned long long)a.add[row] : 0ULL));
    }
}

// ---- single token, streamed: the CTA asks the copy engine for its whole run of tiles up front (one bulk copy per
// tile, each with its own single-use barrier), then multiplies the tiles as they land.  Same arithmetic as the
// kernel above; the weights come from shared memory instead of per-lane loads, so every byte of the run is in
// flight from the first instruction.
constexpr unsigned Q1_WAIT_LIMIT = 1u << 22;     // polls before a wait gives up and raises flag bit 3

__device__ __forceinline__ uint32_t q1_s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool q1_wait(uint64_t *bar) {                       // bounded: false if the bytes never arrived
    for (unsigned it = 0; it < Q1_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(q1_s32(bar)) : "memory");
        if (ok) return true;
    }
    return false;
}

template <int BPW, typename DT>
__global__ void __launch_bounds__(512) q1_stream_kernel(const Q1Args a) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    extern __shared__ __align__(128) uint8_t q1_sm[];
    __shared__ int s_timeout;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long long K = a.nb * 128;
    const long long tile0 = (long long)blockIdx.x * a.tiles_per_cta;
    const int ntile = (int)min((long long)a.tiles_per_cta, a.n_tiles - tile0);
    const uint32_t tile_bytes = (uint32_t)(a.nb * US);
    uint8_t *wbuf = q1_sm;                                                                        // [tiles_per_cta][tile_bytes]
    unsigned long long *red = reinterpret_cast<unsigned long long *>(q1_sm + (size_t)a.tiles_per_cta * tile_bytes);   // [tiles][16]
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + a.tiles_per_cta * 16);
    for (int i = threadIdx.x; i < ntile; i += blockDim.x)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(q1_s32(&bars[i])));
    for (int i = threadIdx.x; i < a.tiles_per_cta * 16; i += blockDim.x) red[i] = 0ULL;
    if (threadIdx.x == 0) s_timeout = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    for (int i = threadIdx.x; i < ntile; i += blockDim.x) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(q1_s32(&bars[i])), "r"(tile_bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(q1_s32(wbuf + (size_t)i * tile_bytes)), "l"(a.units + (size_t)(tile0 + i) * tile_bytes), "r"(tile_bytes),
                       "r"(q1_s32(&bars[i])) : "memory");
    }

    uint32_t bf[BPW][8];
    unsigned long long tot[BPW];
    const int8_t *xcol = a.xl + (long long)col_limb(g) * K + 8 * t;
#pragma unroll
    for (int i = 0; i < BPW; i++) {
        const long long b = warp + (long long)i * W;
        tot[i] = 0;
#pragma unroll
        for (int m = 0; m < 4; m++) { bf[i][2 * m] = 0; bf[i][2 * m + 1] = 0; }
        if (b < a.nb) {
            tot[i] = (unsigned long long)__ldg(a.totals + b);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint2 v = ldg64(xcol + b * 128 + 32 * m);
                bf[i][2 * m] = v.x; bf[i][2 * m + 1] = v.y;
            }
        }
    }
    const int myrow = g + 8 * (t & 1);
    for (int tl = 0; tl < ntile; tl++) {
        if (!q1_wait(&bars[tl])) { s_timeout = 1; break; }
        const uint8_t *tile = wbuf + (size_t)tl * tile_bytes;
        unsigned long long acc = 0;
#pragma unroll
        for (int i = 0; i < BPW; i++) {
            const long long b = warp + (long long)i * W;
            if (b >= a.nb) continue;
            const uint8_t *unit = tile + b * US;
            const uint2 w = *reinterpret_cast<const uint2 *>(unit + lane * 8);
            const int64_t sc = (int64_t)*(reinterpret_cast<const DT *>(unit + 256) + myrow);
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                uint32_t af[4];
                q1_afrag(w, m, af);
                mma_u8s8_k32(c, af[0], af[1], af[2], af[3], bf[i][2 * m], bf[i][2 * m + 1]);
            }
            unsigned long long lo, hi;
            q1_partials(c, t, lo, hi);
            const unsigned long long send = (t & 1) ? lo : hi;
            unsigned long long mine = ((t & 1) ? hi : lo) + __shfl_xor_sync(0xffffffffu, send, 1);
            mine += __shfl_xor_sync(0xffffffffu, mine, 2);
            const unsigned long long s = 2ULL * mine - tot[i];
            acc += (unsigned long long)q1_shift((int64_t)(s * (unsigned long long)sc), a.sh);
        }
        if (t < 2) atomicAdd(&red[tl * 16 + myrow], acc);
    }
    __syncthreads();
    if (s_timeout) {                                       // a copy never arrived: report, store nothing
        if (threadIdx.x == 0 && a.flags) atomicOr(a.flags, 8);
        return;
    }
    for (int i = threadIdx.x; i < ntile * 16; i += blockDim.x) {
        const long long row = tile0 * 16 + i;
        if (row < a.out_f) a.out[row] = (int64_t)(red[i] + (a.add ? (unsigned long long)a.add[row] : 0ULL));
    }
}

// ---- many tokens: one warp per 16-row tile, the expanded bits stay in registers, tokens in groups of four ----
constexpr int Q1_TC = 16;                                             // tokens per CTA

template <typename DT>
__global__ void __launch_bounds__(256, 2) q1_tile_kernel(const Q1Args a) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long long tile = (long long)blockIdx.x * 8 + warp;
    if (tile >= a.n_tiles) return;
    const long long K = a.nb * 128;
    const long long tok0 = (long long)blockIdx.y * Q1_TC;
    const int ngrp = (int)((min((long long)Q1_TC, a.T - tok0) + 3) >> 2);
    unsigned long long acc[Q1_TC / 4][2];
#pragma unroll
    for (int q = 0; q < Q1_TC / 4; q++) { acc[q][0] = 0; acc[q][1] = 0; }

    const uint8_t *unit = a.units + tile * a.nb * US;
    for (long long b = 0; b < a.nb; b++, unit += US) {
        const uint2 w = ldg64(unit + lane * 8);
        const int64_t sc_lo = q1_scale_at<DT>(unit, g), sc_hi = q1_scale_at<DT>(unit, g + 8);
        uint32_t af[4][4];
#pragma unroll
        for (int m = 0; m < 4; m++) q1_afrag(w, m, af[m]);
#pragma unroll
        for (int q = 0; q < Q1_TC / 4; q++) {
            if (q < ngrp) {
                unsigned long long lo[4], hi[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const long long tok = min(tok0 + 4 * q + j, a.T - 1);
                    const int8_t *xp = a.xl + (tok * 8 + col_limb(g)) * K + b * 128 + 8 * t;
                    int c[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int m = 0; m < 4; m++) {
                        const uint2 v = ldg64(xp + 32 * m);
                        mma_u8s8_k32(c, af[m][0], af[m][1], af[m][2], af[m][3], v.x, v.y);
                    }
                    q1_partials(c, t, lo[j], hi[j]);
                }
                // reduce-scatter: lane t ends with the complete sums of token 4q + t (rows g and g + 8)
                const int h = t >> 1;                                       // first exchange keeps tokens 2h, 2h + 1
                unsigned long long kl[2], kh[2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const unsigned long long sl = h ? lo[j] : lo[2 + j], shv = h ? hi[j] : hi[2 + j];
                    kl[j] = (h ? lo[2 + j] : lo[j]) + __shfl_xor_sync(0xffffffffu, sl, 2);
                    kh[j] = (h ? hi[2 + j] : hi[j]) + __shfl_xor_sync(0xffffffffu, shv, 2);
                }
                const int o = t & 1;                                        // second exchange keeps token 2h + o
                const unsigned long long pl = (o ? kl[1] : kl[0]) + __shfl_xor_sync(0xffffffffu, o ? kl[0] : kl[1], 1);
                const unsigned long long ph = (o ? kh[1] : kh[0]) + __shfl_xor_sync(0xffffffffu, o ? kh[0] : kh[1], 1);
                const long long tok = min(tok0 + 4 * q + t, a.T - 1);
                const unsigned long long tt = (unsigned long long)__ldg(a.totals + tok * a.nb + b);
                acc[q][0] += (unsigned long long)q1_shift((int64_t)((2ULL * pl - tt) * (unsigned long long)sc_lo), a.sh);
                acc[q][1] += (unsigned long long)q1_shift((int64_t)((2ULL * ph - tt) * (unsigned long long)sc_hi), a.sh);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < Q1_TC / 4; q++) {
        const long long tok = tok0 + 4 * q + t;
        if (q < ngrp && tok < a.T) {
            const long long row = tile * 16 + g;
            if (row < a.out_f)
                a.out[tok * a.out_f + row] = (int64_t)(acc[q][0] + (a.add ? (unsigned long long)a.add[tok * a.out_f + row] : 0ULL));
            if (row + 8 < a.out_f)
                a.out[tok * a.out_f + row + 8] = (int64_t)(acc[q][1] + (a.add ? (unsigned long long)a.add[tok * a.out_f + row + 8] : 0ULL));
        }
    }
}

template <int BPW, typename DT>
cudaError_t launch_gemv(const Q1Args &a_in, int W, cudaStream_t s) {
    Q1Args a = a_in;
    int sms = 148;
    const long long target = 4LL * sms;              // several CTAs per SM: one's loads overlap another's multiplies
    a.tiles_per_cta = (int)std::max<long long>(1, (a.n_tiles + target - 1) / target);
    const unsigned grid = (unsigned)((a.n_tiles + a.tiles_per_cta - 1) / a.tiles_per_cta);
    q1_gemv_kernel<BPW, DT><<<grid, 32 * W, (size_t)a.tiles_per_cta * 16 * sizeof(unsigned long long), s>>>(a);
    note_launch();
    return cudaGetLastError();
}

int g_q1_stream = 0;               // 1: single-token products through the bulk-copy kernel (same speed: the arithmetic per unit bounds both)

template <int BPW, typename DT>
cudaError_t launch_q1_stream(const Q1Args &a_in, int W, cudaStream_t s) {
    Q1Args a = a_in;
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    const size_t tile_bytes = (size_t)a.nb * US, per_tile = tile_bytes + 16 * 8 + 8;
    const int max_tpc = (int)((200 * 1024) / per_tile);
    if (max_tpc < 1) return cudaErrorInvalidConfiguration;
    int tpc = (int)((a.n_tiles + 147) / 148);                    // one wave when the run fits in shared memory
    if (tpc > max_tpc) tpc = max_tpc;
    a.tiles_per_cta = tpc;
    const unsigned grid = (unsigned)((a.n_tiles + tpc - 1) / tpc);
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(q1_stream_kernel<BPW, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    q1_stream_kernel<BPW, DT><<<grid, 32 * W, (size_t)tpc * per_tile + 16, s>>>(a);
    note_launch();
    return cudaGetLastError();
}

template <typename DT>
cudaError_t launch_apply_t(const Q1Args &a, cudaStream_t s) {
    if (a.T == 1 && a.nb <= 128 && g_q1_stream) {
        const int W = a.nb > 64 ? 16 : 8;
        const int bpw = (int)((a.nb + W - 1) / W);
        if (bpw <= 2) return launch_q1_stream<2, DT>(a, W, s);
        if (bpw <= 4) return launch_q1_stream<4, DT>(a, W, s);
        if (bpw <= 6) return launch_q1_stream<6, DT>(a, W, s);
        return launch_q1_stream<8, DT>(a, W, s);
    }
    if (a.T == 1 && a.nb <= 128) {
        const int W = a.nb > 64 ? 16 : 8;
        const int bpw = (int)((a.nb + W - 1) / W);
        if (bpw <= 2) return launch_gemv<2, DT>(a, W, s);
        if (bpw <= 4) return launch_gemv<4, DT>(a, W, s);
        if (bpw <= 6) return launch_gemv<6, DT>(a, W, s);
        return launch_gemv<8, DT>(a, W, s);
    }
    dim3 grid((unsigned)((a.n_tiles + 7) / 8), (unsigned)((a.T + Q1_TC - 1) / Q1_TC));
    q1_tile_kernel<DT><<<grid, 256, 0, s>>>(a);
    note_launch();
    return cudaGetLastError();
}

// SiLU(gate) * up with the wrapping products of bonsai/src/trinote/infer_int/reference_bonsai.py:246-262,611-614:
// silu = (gate * sigmoid(gate)) >> frac and h = (silu * up) >> frac, both products modulo 2^64.
__global__ void q1_silu_mul_kernel(const int64_t *gate, const int64_t *up, long long n, int frac, int64_t log2e, int64_t clip,
                                   int64_t *out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t g = gate[i];
    const int64_t sg = sigmoid_fixed_c(g, frac, log2e, clip);
    const int64_t silu = (int64_t)((unsigned long long)g * (unsigned long long)sg) >> frac;
    out[i] = (int64_t)((unsigned long long)silu * (unsigned long long)up[i]) >> frac;
}

// one row of a registered Q1_0 matrix as int64: sign * block scale (reference_bonsai.py:138-146 q1_rows_fp)
template <typename DT>
__global__ void q1_embed_row_kernel(const uint8_t *units, long long nb, const int *row_dev, long long row_host, int64_t *out) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    const long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= nb * 128) return;
    const long long row = row_dev ? (long long)*row_dev : row_host, b = k >> 7;
    const int kk = (int)(k & 127), rloc = (int)(row & 15), g = rloc & 7, hi = rloc >> 3;
    const int m = kk >> 5, t = (kk & 31) >> 3, jj = ((kk & 31) >> 2) & 1, i = kk & 3;
    const int r = (m & 1) * 4 + ((jj << 1) | hi), mp = m >> 1;
    const uint8_t *unit = units + ((row >> 4) * nb + b) * US;
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(unit) + (4 * g + t) * 2 + mp);
    const int64_t sc = (int64_t)__ldg(reinterpret_cast<const DT *>(unit + 256) + rloc);
    out[k] = ((w >> (r + 8 * i)) & 1u) ? sc : -sc;
}

}  // namespace

void set_q1_stream(int on) { g_q1_stream = on ? 1 : 0; }

size_t q1_unit_bytes(bool sc32) { return 256 + 16 * (sc32 ? 4 : 8); }

cudaError_t launch_q1_repack(const uint8_t *bits, const void *scale, int src_bits, bool sc32, long long out_f, long long nb,
                             uint8_t *units, cudaStream_t s) {
    const long long n_tiles = (out_f + 15) / 16, n = n_tiles * nb * 80;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (src_bits == 64 && !sc32) q1_repack_kernel<long long, long long><<<grid, 256, 0, s>>>(bits, (const long long *)scale, out_f, nb, n_tiles, units);
    else if (src_bits == 64) q1_repack_kernel<long long, int><<<grid, 256, 0, s>>>(bits, (const long long *)scale, out_f, nb, n_tiles, units);
    else if (sc32) q1_repack_kernel<int, int><<<grid, 256, 0, s>>>(bits, (const int *)scale, out_f, nb, n_tiles, units);
    else return cudaErrorInvalidValue;
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_q1_prep(const int64_t *x, long long T, long long nb, int8_t *planes, int64_t *totals, int *nl_out, cudaStream_t s) {
    const long long warps = T * nb;
    q1_prep_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, s>>>(x, nullptr, 0, 0, 0, 0, T, nb, planes, totals, nl_out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_q1_prep_swiglu(const int64_t *gate, const int64_t *up, long long ld, int frac, long long T, long long nb,
                                  int8_t *planes, int64_t *totals, cudaStream_t s) {
    if (!gate || !up || frac < 1 || frac > 29) return cudaErrorInvalidValue;
    const long long warps = T * nb;
    q1_prep_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, s>>>(gate, up, ld, frac, sigmoid_log2e(frac), sigmoid_clip(frac), T, nb,
                                                                        planes, totals, nullptr);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_q1_apply(const uint8_t *units, bool sc32, long long out_f, long long nb, const int8_t *planes,
                            const int64_t *totals, long long T, long long frac, int64_t *out, cudaStream_t s, const int64_t *add) {
    if (out_f <= 0 || nb <= 0 || T <= 0) return cudaErrorInvalidValue;
    Q1Args a;
    a.units = units; a.out_f = out_f; a.nb = nb; a.n_tiles = (out_f + 15) / 16; a.T = T;
    a.sh = frac <= 0 ? 0 : (frac >= 63 ? 63 : (int)frac);
    a.tiles_per_cta = 1; a.xl = planes; a.totals = totals; a.out = out; a.add = add; a.flags = shared_flag_word();
    return sc32 ? launch_apply_t<int>(a, s) : launch_apply_t<long long>(a, s);
}

cudaError_t launch_q1_silu_mul(const int64_t *gate, const int64_t *up, long long n, int frac, int64_t *out, cudaStream_t s) {
    if (n <= 0 || frac < 1 || frac > 29) return cudaErrorInvalidValue;
    q1_silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, n, frac, sigmoid_log2e(frac), sigmoid_clip(frac), out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_q1_embed_row(const uint8_t *units, bool sc32, long long nb, const int *row_dev, long long row_host, int64_t *out,
                                cudaStream_t s) {
    const unsigned grid = (unsigned)((nb * 128 + 255) / 256);
    if (sc32) q1_embed_row_kernel<int><<<grid, 256, 0, s>>>(units, nb, row_dev, row_host, out);
    else q1_embed_row_kernel<long long><<<grid, 256, 0, s>>>(units, nb, row_dev, row_host, out);
    note_launch();
    return cudaGetLastError();
}

}  // namespace iie
