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
#include <cuda.h>

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
    const int *nl_dev;              // tcgen05 tiles: digit planes in use by xl (planes at and above it are zero), on the device
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


// ---- many tokens on the 5th-generation tensor cores ------------------------------------------------------------------------
// Tile: 128 weight rows (MMA M, TMEM lanes) x 64 tokens (MMA N) x one 128-weight block at a time.  A = the block's sign bits
// expanded to bytes 0/1 (u8) in the canonical K-major layout, written by eight warps straight from the repacked units (a
// shift and a mask give four consecutive columns of a row); B = the eight digit planes of the 64 tokens (s8), fetched by
// the copy engine (TMA, 64-byte swizzle) from the [token][8][K] planes; one TMEM accumulator per digit plane (8 x 64 = all 512
// columns).  After the 32 MMAs of a block the eight warps read the accumulators out: P = sum_l 256^l acc_l (mod 2^64),
// (2 P - S) * scale, the per-block floor shift, added into 64-bit registers (a thread owns one row and 32 tokens);
// the issuer waits for that before it starts the next block, the producers are a block ahead.  Every wait is bounded; the
// eight warps leave the block loop by a vote.
constexpr int QT_PRODUCERS = 256, QT_THREADS = QT_PRODUCERS + 32, QT_STAGES = 4, QT_N = 64;
constexpr int QT_A_BYTES = 128 * 64, QT_B_PLANE = QT_N * 64, QT_STAGE = QT_A_BYTES + 8 * QT_B_PLANE;      // 8192 + 32768
constexpr unsigned QT_WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t qt_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool qt_wait(uint64_t *b, uint32_t parity, volatile int *abort_flag) {
    for (unsigned it = 0; it < QT_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(qt_u32(b)), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ bool qt_all_ok(bool ok) {                // AND over the producer warps (named barrier 1)
    uint32_t r;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 q, %1, 0;\n barrier.cta.red.and.pred p, 1, %2, q;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(r) : "r"((uint32_t)ok), "r"(QT_PRODUCERS) : "memory");
    return r != 0;
}

// digit planes in use: one warp per (token, plane) row of the [T][8][K] planes ORs the row; a non-zero row of plane l
// raises the cell to l + 1 (the cell is cleared before the launch)
__device__ int d_q1_nl;
__global__ void __launch_bounds__(256) q1_planes_in_use_kernel(const int8_t *__restrict__ planes, long long rows, long long K, int *cell) {
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= rows) return;
    const int lane = threadIdx.x & 31, l = (int)(wid & 7);
    if (l == 0) return;                                            // one plane is always in use
    const uint4 *src = reinterpret_cast<const uint4 *>(planes + wid * K);
    uint32_t any = 0;
    for (long long i = lane; i < K / 16; i += 32) { const uint4 v = __ldg(src + i); any |= v.x | v.y | v.z | v.w; }
    any = __reduce_or_sync(0xffffffffu, any);
    if (lane == 0 && any) atomicMax(cell, l + 1);
}

template <typename DT>
__global__ void __launch_bounds__(QT_THREADS, 1) q1_tc_kernel(const Q1Args a, const __grid_constant__ CUtensorMap xmap) {
    constexpr int US = 256 + 16 * (int)sizeof(DT);
    extern __shared__ __align__(1024) unsigned char qt_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(qt_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[QT_STAGES], empty_bar[QT_STAGES], acc_bar, free_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    long long *s_tot = reinterpret_cast<long long *>(smem + (size_t)QT_STAGES * QT_STAGE);      // block sums of the tile's tokens [nb][64]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long tile = blockIdx.x, tok0 = (long long)blockIdx.y * QT_N;          // 128-row tile, first token
    const int nb = (int)a.nb, n_chunks = 2 * nb;
    const int nl = max(1, min(8, *a.nl_dev));                       // digit planes that are not all zero (uniform over the grid)
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < QT_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(qt_u32(&full_bar[s])), "r"(QT_PRODUCERS / 32 + 1));   // the producer warps + the copy's expect_tx arrival
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(qt_u32(&empty_bar[s])), "r"(1));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(qt_u32(&acc_bar)), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(qt_u32(&free_bar)), "r"(QT_PRODUCERS / 32));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == QT_PRODUCERS / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(qt_u32(&s_tmem)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    for (int i = tid; i < nb * QT_N; i += QT_THREADS) {            // s_tot[b][token]
        const int b = i / QT_N, tk = i - b * QT_N;
        s_tot[i] = a.totals[min(tok0 + tk, a.T - 1) * nb + b];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp < QT_PRODUCERS / 32) {
        // ---- producer part: thread -> (16-row sub-tile, lane (g, t) of the unit's bit words): one word, eight bit groups -------
        const int sub = tid >> 5, ul = tid & 31, g = ul >> 2, t = ul & 3;
        const long long tile16 = tile * 8 + sub;
        const bool sub_ok = tile16 < a.n_tiles;
        const int np_t = nl <= 3 ? 3 : nl == 4 ? 4 : nl <= 6 ? 6 : 8;        // planes fetched, multiplied and read out
        auto words = [&](int b) {                                  // this thread's two bit words of block b (one per chunk)
            return sub_ok ? ldg64(a.units + (tile16 * nb + b) * US + ul * 8) : make_uint2(0u, 0u);
        };
        auto produce = [&](int c, uint32_t w) {                    // chunk c = half (c & 1) of block c >> 1, w = its bit word
            const int s = c % QT_STAGES;
            if (c >= QT_STAGES && !qt_wait(&empty_bar[s], ((c / QT_STAGES) - 1) & 1, &s_abort)) return false;
            unsigned char *stage = smem + (size_t)s * QT_STAGE;
            if (tid == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(qt_u32(&full_bar[s])), "r"(np_t * QT_B_PLANE) : "memory");
#pragma unroll
                for (int l = 0; l < 8; l++)
                    if (l < np_t) asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                                 ::"r"(qt_u32(stage + QT_A_BYTES + l * QT_B_PLANE)), "l"(reinterpret_cast<uint64_t>(&xmap)), "r"(c * 64), "r"(l),
                                   "r"((int)tok0), "r"(qt_u32(&full_bar[s])) : "memory");
            }
#pragma unroll
            for (int r = 0; r < 8; r++) {                          // bit group r: MMA m & 1 = rhalf, column half jj, row half hi
                const int rhalf = r >> 2, jj = (r >> 1) & 1, hi = r & 1;
                const int row = sub * 16 + g + 8 * hi;
                const int k16 = 2 * rhalf + (t >> 1), kin = 8 * (t & 1) + 4 * jj;              // columns 32 rhalf + 8 t + 4 jj + (0..3) of the chunk
                *reinterpret_cast<uint32_t *>(stage + k16 * (128 * 16) + (row >> 3) * 128 + (row & 7) * 16 + kin) = (w >> r) & 0x01010101u;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qt_u32(&full_bar[s])) : "memory");
            return true;
        };
        // ---- read-out part: TMEM lane = row of the tile, 32 tokens per thread ------------------------------------------
        const int rowt = (warp & 3) * 32 + lane, cg = warp >> 2;
        const long long row = tile * 128 + rowt;
        const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const bool row_ok = row < a.out_f && (tile * 8 + (rowt >> 4)) < a.n_tiles;
        const uint8_t *scale_unit = a.units + ((tile * 8 + (rowt >> 4)) * (long long)nb) * US;
        unsigned long long acc64[32];
#pragma unroll
        for (int j = 0; j < 32; j++) acc64[j] = 0;
        // read-out of one block with NP planes known at compile time (NP >= nl: the planes between are zero and multiplied):
        // eight tokens per round; TMEM is handed back as soon as the last round's loads have landed, before its arithmetic
        auto drain = [&](auto np_c, int b, unsigned long long sc) {
            constexpr int NP = decltype(np_c)::value;
            const long long *tot = s_tot + b * QT_N + cg * 32;
#pragma unroll
            for (int ro = 0; ro < 4; ro++) {
                int r[NP][8];
#pragma unroll
                for (int l = 0; l < NP; l++)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[l][0]), "=r"(r[l][1]), "=r"(r[l][2]), "=r"(r[l][3]), "=r"(r[l][4]), "=r"(r[l][5]), "=r"(r[l][6]), "=r"(r[l][7])
                                 : "r"(tlane + l * QT_N + cg * 32 + ro * 8));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ro == 3) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qt_u32(&free_bar)) : "memory");
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // P = sum_l 256^l acc_l (mod 2^64): four planes at a time as 32 x 32 -> 64 multiply-adds
                    long long lo = (long long)r[0][j];
#pragma unroll
                    for (int l = 1; l < 4 && l < NP; l++) lo += (long long)r[l][j] * (long long)(1 << (8 * l));
                    unsigned long long P = (unsigned long long)lo;
                    if (NP > 4) {
                        long long hi4 = (long long)r[4][j];
#pragma unroll
                        for (int l = 5; l < NP; l++) hi4 += (long long)r[l][j] * (long long)(1 << (8 * (l - 4)));
                        P += (unsigned long long)hi4 << 32;
                    }
                    acc64[ro * 8 + j] += (unsigned long long)q1_shift((int64_t)((2ULL * P - (unsigned long long)tot[ro * 8 + j]) * sc), a.sh);
                }
            }
        };
        uint2 wn = words(0);
        bool ok = produce(0, wn.x) && produce(1, wn.y);
        if (nb > 1) wn = words(1);
        for (int b = 0; b < nb; b++) {
            if (ok && b + 1 < nb) ok = produce(2 * b + 2, wn.x) && produce(2 * b + 3, wn.y);
            if (b + 2 < nb) wn = words(b + 2);                     // in flight during the wait and the read-out
            const unsigned long long sc = row_ok ? (unsigned long long)q1_scale_at<DT>(scale_unit + (long long)b * US, rowt & 15) : 0ULL;   // in flight during the wait
            ok = ok && qt_wait(&acc_bar, b & 1, &s_abort);
            if (!qt_all_ok(ok)) break;                             // uniform over the producer warps
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (nl <= 3) drain(std::integral_constant<int, 3>{}, b, sc);
            else if (nl == 4) drain(std::integral_constant<int, 4>{}, b, sc);
            else if (nl <= 6) drain(std::integral_constant<int, 6>{}, b, sc);
            else drain(std::integral_constant<int, 8>{}, b, sc);
        }
        if (ok && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const long long tok = tok0 + cg * 32 + j;
                if (tok < a.T) a.out[tok * a.out_f + row] = (int64_t)(acc64[j] + (a.add ? (unsigned long long)a.add[tok * a.out_f + row] : 0ULL));
            }
        }
    } else {
        // ---- MMA issuer ---------------------------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC = (2u << 4) | (1u << 10) | ((uint32_t)(QT_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);     // u8 x s8 -> s32
            const int np = nl <= 3 ? 3 : nl == 4 ? 4 : nl <= 6 ? 6 : 8;      // the planes the read-out combines
            bool ok = true;
            for (int c = 0; c < n_chunks && ok; c++) {
                const int s = c % QT_STAGES;
                ok = qt_wait(&full_bar[s], (c / QT_STAGES) & 1, &s_abort);
                if (ok && (c & 1) == 0 && c > 0) ok = qt_wait(&free_bar, ((c >> 1) - 1) & 1, &s_abort);      // the previous block has left TMEM
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t stage = qt_u32(smem + (size_t)s * QT_STAGE);
                // A: K-major, no swizzle (LBO = distance of the two 16-byte K halves of an MMA, SBO = 8-row groups); B: 64-byte swizzle
                const uint64_t da0 = (uint64_t)((stage >> 4) & 0x3FFF) | ((uint64_t)((128 * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | (1ULL << 46);
                const uint64_t db0 = (uint64_t)(((stage + QT_A_BYTES) >> 4) & 0x3FFF) | (1ULL << 16) | ((uint64_t)(512 >> 4) << 32) | (1ULL << 46) | (4ULL << 61);
#pragma unroll
                for (int ks = 0; ks < 2; ks++)
#pragma unroll
                    for (int l = 0; l < 8; l++) {
                        if (l >= np) continue;
                        const uint64_t da = da0 + (uint64_t)((ks * 2 * 128 * 16) >> 4);
                        const uint64_t db = db0 + (uint64_t)((l * QT_B_PLANE + ks * 32) >> 4);
                        const uint32_t accumulate = ((c & 1) == 0 && ks == 0) ? 0u : 1u;      // a block starts from zero
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                                     ::"r"(tmem + l * QT_N), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u) : "memory");
                    }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(qt_u32(&empty_bar[s])) : "memory");
                if (c & 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(qt_u32(&acc_bar)) : "memory");
            }
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == QT_PRODUCERS / 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
    if (tid == 0 && s_abort && a.flags) atomicOr(a.flags, 8);
}

using QtEncode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
QtEncode qt_encode() {
    static QtEncode fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<QtEncode>(p);
    }();
    return fn;
}

int g_q1_tc = 1;                   // 1: products of 32 tokens or more on the tcgen05 tiles, 0: always the warp-MMA tiles

template <typename DT>
cudaError_t launch_q1_tc(const Q1Args &a_in, cudaStream_t s) {
    QtEncode enc = qt_encode();
    if (!enc) return cudaErrorNotSupported;
    Q1Args a = a_in;
    const long long K = a.nb * 128;
    static int *cell = nullptr;
    if (!cell && cudaGetSymbolAddress((void **)&cell, d_q1_nl) != cudaSuccess) return cudaErrorNotSupported;
    if (cudaMemsetAsync(cell, 0, sizeof(int), s) != cudaSuccess) return cudaGetLastError();
    q1_planes_in_use_kernel<<<(unsigned)((a.T * 8 * 32 + 255) / 256), 256, 0, s>>>(a.xl, a.T * 8, K, cell);
    note_launch();
    a.nl_dev = cell;
    CUtensorMap map;
    const cuuint64_t dims[3] = {(cuuint64_t)K, 8, (cuuint64_t)a.T};
    const cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)(8 * K)};
    const cuuint32_t box[3] = {64, 1, QT_N}, estr[3] = {1, 1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t *>(a.xl), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    if (a.nb > 128) return cudaErrorNotSupported;                  // the block sums of a tile's tokens sit in shared memory
    const size_t smem = (size_t)QT_STAGES * QT_STAGE + (size_t)a.nb * QT_N * 8 + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(q1_tc_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)QT_STAGES * QT_STAGE + (size_t)128 * QT_N * 8 + 1024));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    dim3 grid((unsigned)((a.out_f + 127) / 128), (unsigned)((a.T + QT_N - 1) / QT_N));
    q1_tc_kernel<DT><<<grid, QT_THREADS, smem, s>>>(a, map);
    note_launch();
    return cudaGetLastError();
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
    if (g_q1_tc && a.T >= 32 && (a.nb * 128) % 16 == 0 && (reinterpret_cast<uintptr_t>(a.xl) & 15) == 0) {
        const cudaError_t e = launch_q1_tc<DT>(a, s);
        if (e == cudaSuccess) return e;
        cudaGetLastError();                                    // no tensor map on this driver: the warp-MMA tiles
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
void set_q1_tc(int on) { g_q1_tc = on ? 1 : 0; }

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
    a.tiles_per_cta = 1; a.xl = planes; a.totals = totals; a.out = out; a.add = add; a.flags = shared_flag_word(); a.nl_dev = nullptr;
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
