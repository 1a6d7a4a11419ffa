// Streamed fused-dequant integer products for the decode / small-batch regime (sm_100a).
//
// Replaces the reference's one-thread-per-output row streamers (north-mini-code/tools/
// nmc_qk_cuda.cu:113-175 dot_q4k/dot_q6k, :222-229 matmul_multi_k, :208-218 silu_k/mul_shift_k,
// :231-237 combine_k) with one kernel family that
//   * streams the repacked blocks with coalesced 128-bit loads (see layout.cuh),
//   * unpacks the 4/6-bit codes in registers into tensor-core A fragments,
//   * multiplies them with the eight balanced base-256 limb planes of the int64 activations
//     (the limbs are the N=8 columns of a warp MMA, so a single pass is exact for any |x| up to
//     127*(2^64-1)/255),
//   * applies the sub-block scales / minimums in int32, the block scale in int64, recombines the
//     limb columns in 128 bits and performs the single floor shift of the reference,
//   * and fuses the neighbouring element-wise steps: integer SiLU * up for the gate/up pair and
//     gate-weighted accumulation for the down projection.
//
// Exactness envelope of the fast path (checked by the host before launch):
//   Q4_K: n_blocks * (max|d_q| * 2^25 + max|dmin_q| * 2^21) < 2^62,  Q6_K: n_blocks * max|d_q| * 2^28 < 2^62.
// Inside it every partial sum below fits its type:
//   Q4_K sub-block dot |S| <= 32*15*128, block sum |T| <= 8*63*|S| < 2^25, minimum term < 2^21;
//   Q6_K sub-block dot |S| <= 16*32*128, block sum |T| <= 16*128*|S| = 2^27.
#include "kernels.h"
#include "layout.cuh"

namespace iie {

namespace {

constexpr int MAX_KSPLIT = 8;   // warps per CTA that share one 16-row tile along K

template <int NTC>
struct Acc {
    int64_t v[NTC][4];          // [pair][c-fragment element]: (row g, col 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
};

__device__ __forceinline__ int sbyte(uint32_t w, int i) { return (int)(w << (24 - 8 * i)) >> 24; }
__device__ __forceinline__ int ubyte(uint32_t w, int i) { return (int)((w >> (8 * i)) & 0xFF); }

// One Q4_K half-tile-block pair (rows g of unit A, rows g of unit B -> MMA rows g and g+8).
template <int NTC>
__device__ __forceinline__ void block_q4k(const uint8_t *ua, const uint8_t *ub, int lane, int fw,
                                          const int8_t *const (&xp)[NTC], int npairs, long long K, long long kbase,
                                          Acc<NTC> &acc) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 qa0 = ldg128_stream(ua + lane * 16), qa1 = ldg128_stream(ua + 512 + lane * 16);
    const uint4 qb0 = ldg128_stream(ub + lane * 16), qb1 = ldg128_stream(ub + 512 + lane * 16);
    const uint4 ma = ldg128(ua + 1024 + g * 16), mb = ldg128(ub + 1024 + g * 16);
    uint32_t scA_lo, scA_hi, mnA_lo, mnA_hi, scB_lo, scB_hi, mnB_lo, mnB_hi;
    q4k_scales(ma.y, ma.z, ma.w, scA_lo, scA_hi, mnA_lo, mnA_hi);
    q4k_scales(mb.y, mb.z, mb.w, scB_lo, scB_hi, mnB_lo, mnB_hi);
    const int64_t dqA = half_to_fixed(ma.x & 0xFFFF, fw), dmA = half_to_fixed(ma.x >> 16, fw);
    const int64_t dqB = half_to_fixed(mb.x & 0xFFFF, fw), dmB = half_to_fixed(mb.x >> 16, fw);
    const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};

    int T4[NTC][4], M4[NTC][4];
#pragma unroll
    for (int p = 0; p < NTC; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) { T4[p][i] = 0; M4[p][i] = 0; }

#pragma unroll
    for (int G = 0; G < 4; G++) {
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            const int j = 2 * G + hi;                       // sub-block index
            const int sh = hi * 4;
            const uint32_t a0 = (wa[2 * G] >> sh) & 0x0f0f0f0fu, a2 = (wa[2 * G + 1] >> sh) & 0x0f0f0f0fu;
            const uint32_t a1 = (wb[2 * G] >> sh) & 0x0f0f0f0fu, a3 = (wb[2 * G + 1] >> sh) & 0x0f0f0f0fu;
            const int scA = ubyte(j < 4 ? scA_lo : scA_hi, j & 3), scB = ubyte(j < 4 ? scB_lo : scB_hi, j & 3);
            const uint32_t mA = (uint32_t)ubyte(j < 4 ? mnA_lo : mnA_hi, j & 3) * 0x01010101u;
            const uint32_t mB = (uint32_t)ubyte(j < 4 ? mnB_lo : mnB_hi, j & 3) * 0x01010101u;
            const long long koff = kbase + 32 * j + 8 * t;
#pragma unroll
            for (int p = 0; p < NTC; p++) {
                if (p < npairs) {
                    const uint2 b = ldg64(xp[p] + (long long)g * K + koff);
                    int c[4] = {0, 0, 0, 0};
                    mma_u8s8_k32(c, a0, a1, a2, a3, b.x, b.y);
                    T4[p][0] += scA * c[0]; T4[p][1] += scA * c[1];
                    T4[p][2] += scB * c[2]; T4[p][3] += scB * c[3];
                    mma_u8s8_k32(M4[p], mA, mB, mA, mB, b.x, b.y);
                }
            }
        }
    }
#pragma unroll
    for (int p = 0; p < NTC; p++) {
        acc.v[p][0] += dqA * T4[p][0] - dmA * M4[p][0];
        acc.v[p][1] += dqA * T4[p][1] - dmA * M4[p][1];
        acc.v[p][2] += dqB * T4[p][2] - dmB * M4[p][2];
        acc.v[p][3] += dqB * T4[p][3] - dmB * M4[p][3];
    }
}

template <int NTC>
__device__ __forceinline__ void block_q6k(const uint8_t *ua, const uint8_t *ub, int lane, int fw,
                                          const int8_t *const (&xp)[NTC], int npairs, long long K, long long kbase,
                                          Acc<NTC> &acc) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 la0 = ldg128_stream(ua + lane * 16), la1 = ldg128_stream(ua + 512 + lane * 16);
    const uint4 ha = ldg128_stream(ua + 1024 + lane * 16);
    const uint4 lb0 = ldg128_stream(ub + lane * 16), lb1 = ldg128_stream(ub + 512 + lane * 16);
    const uint4 hb = ldg128_stream(ub + 1024 + lane * 16);
    const uint4 sa = ldg128(ua + 1536 + g * 16), sb = ldg128(ub + 1536 + g * 16);
    const uint32_t da = __ldg(reinterpret_cast<const unsigned short *>(ua + 1664 + g * 2));
    const uint32_t db = __ldg(reinterpret_cast<const unsigned short *>(ub + 1664 + g * 2));
    const int64_t dqA = half_to_fixed(da, fw), dqB = half_to_fixed(db, fw);
    const uint32_t lA[8] = {la0.x, la0.y, la0.z, la0.w, la1.x, la1.y, la1.z, la1.w};   // [h][u]{A,B}
    const uint32_t lB[8] = {lb0.x, lb0.y, lb0.z, lb0.w, lb1.x, lb1.y, lb1.z, lb1.w};
    const uint32_t hA[4] = {ha.x, ha.y, ha.z, ha.w}, hB[4] = {hb.x, hb.y, hb.z, hb.w};  // [h*2+u]
    const uint32_t sA[4] = {sa.x, sa.y, sa.z, sa.w}, sB[4] = {sb.x, sb.y, sb.z, sb.w};  // 16 int8 scales

    int T4[NTC][4];
#pragma unroll
    for (int p = 0; p < NTC; p++)
#pragma unroll
        for (int i = 0; i < 4; i++) T4[p][i] = 0;

#pragma unroll
    for (int h = 0; h < 2; h++) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t wAa = lA[(h * 2 + u) * 2], wAb = lA[(h * 2 + u) * 2 + 1], wAh = hA[h * 2 + u];
            const uint32_t wBa = lB[(h * 2 + u) * 2], wBb = lB[(h * 2 + u) * 2 + 1], wBh = hB[h * 2 + u];
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {
                // weight 128h + 32kq + 16u + 4t + i: low nibble source word and 2-bit field kq of the high word
                const uint32_t nA = (kq & 1) ? wAb : wAa, nB = (kq & 1) ? wBb : wBa;
                const uint32_t loA = (kq < 2 ? nA : (nA >> 4)) & 0x0f0f0f0fu, loB = (kq < 2 ? nB : (nB >> 4)) & 0x0f0f0f0fu;
                const uint32_t hiA = ((wAh >> (2 * kq)) << 4) & 0x30303030u, hiB = ((wBh >> (2 * kq)) << 4) & 0x30303030u;
                const uint32_t qA = __vsub4(loA | hiA, 0x20202020u), qB = __vsub4(loB | hiB, 0x20202020u);
                const int si = 8 * h + 2 * kq + u;
                const int scA = sbyte(sA[si >> 2], si & 3), scB = sbyte(sB[si >> 2], si & 3);
                const long long koff = kbase + 128 * h + 32 * kq + 16 * u + 4 * t;
#pragma unroll
                for (int p = 0; p < NTC; p++) {
                    if (p < npairs) {
                        const uint32_t b = ldg32(xp[p] + (long long)g * K + koff);
                        int c[4] = {0, 0, 0, 0};
                        mma_s8s8_k16(c, qA, qB, b);
                        T4[p][0] += scA * c[0]; T4[p][1] += scA * c[1];
                        T4[p][2] += scB * c[2]; T4[p][3] += scB * c[3];
                    }
                }
            }
        }
    }
#pragma unroll
    for (int p = 0; p < NTC; p++) {
        acc.v[p][0] += dqA * T4[p][0]; acc.v[p][1] += dqA * T4[p][1];
        acc.v[p][2] += dqB * T4[p][2]; acc.v[p][3] += dqB * T4[p][3];
    }
}

// Recombine the eight limb columns of one output row: sum_c col[c] * 256^c, floor-shift by fw.
__device__ __forceinline__ int64_t recombine(const unsigned long long *cols, int fw) {
    i128 v = 0;
#pragma unroll
    for (int c = 7; c >= 0; c--) v = (v << 8) + (i128)(int64_t)cols[c];
    return (int64_t)(v >> fw);
}

template <int QT, int MODE, int NTC>
__global__ void __launch_bounds__(32 * MAX_KSPLIT) skinny_kernel(const SkinnyArgs a) {
    __shared__ unsigned long long red[NTC][16][8];
    const int grp = blockIdx.y;
    const int expert = a.grp_expert ? a.grp_expert[grp] : grp;
    const int p_lo = a.grp_off ? a.grp_off[grp] : grp * a.pairs_per_group;
    const int p_hi = a.grp_off ? a.grp_off[grp + 1] : p_lo + a.pairs_per_group;
    if (p_lo >= p_hi) return;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const long long nb = a.n_blocks, K = nb * 256;
    const long long n_ht = (a.out_f + 7) >> 3;
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    long long htA, htB;
    const uint8_t *baseA = a.wa[expert], *baseB;
    if (MODE == MODE_GATEUP) { htA = htB = blockIdx.x; baseB = a.wb[expert]; }
    else { htA = 2LL * blockIdx.x; htB = htA + 1 < n_ht ? htA + 1 : htA; baseB = baseA; }
    const uint8_t *ua0 = baseA + htA * nb * HTB, *ub0 = baseB + htB * nb * HTB;

    for (int p0 = p_lo; p0 < p_hi; p0 += NTC) {
        const int npairs = min(NTC, p_hi - p0);
        for (int i = threadIdx.x; i < NTC * 16 * 8; i += blockDim.x) (&red[0][0][0])[i] = 0ULL;
        __syncthreads();

        const int8_t *xp[NTC];
#pragma unroll
        for (int p = 0; p < NTC; p++) {
            const int pr = p0 + (p < npairs ? p : 0);
            const long long xrow = a.xidx ? a.xidx[pr] : pr;
            xp[p] = a.xl + xrow * 8 * K;
        }
        Acc<NTC> acc;
#pragma unroll
        for (int p = 0; p < NTC; p++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc.v[p][i] = 0;

        for (long long b = warp; b < nb; b += nwarps) {
            if (QT == QT_Q4K) block_q4k<NTC>(ua0 + b * HTB, ub0 + b * HTB, lane, a.fw, xp, npairs, K, b * 256, acc);
            else              block_q6k<NTC>(ua0 + b * HTB, ub0 + b * HTB, lane, a.fw, xp, npairs, K, b * 256, acc);
        }
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int p = 0; p < NTC; p++) {
            if (p < npairs) {
                atomicAdd(&red[p][g][2 * t], (unsigned long long)acc.v[p][0]);
                atomicAdd(&red[p][g][2 * t + 1], (unsigned long long)acc.v[p][1]);
                atomicAdd(&red[p][g + 8][2 * t], (unsigned long long)acc.v[p][2]);
                atomicAdd(&red[p][g + 8][2 * t + 1], (unsigned long long)acc.v[p][3]);
            }
        }
        __syncthreads();

        if (MODE == MODE_GATEUP) {
            // rows 0..7 are the gate projection, rows 8..15 the up projection of the same output index
            for (int idx = threadIdx.x; idx < npairs * 8; idx += blockDim.x) {
                const int p = idx >> 3, r = idx & 7;
                const long long row = htA * 8 + r;
                if (row < a.out_f) {
                    const int64_t yg = recombine(red[p][r], a.fw), yu = recombine(red[p][r + 8], a.fw);
                    const int64_t gu = mul_shift(silu_fixed(yg, a.fa), yu, a.fa);
                    const long long pr = p0 + p;
                    if (a.out) a.out[pr * a.out_f + row] = gu;
                    if (a.out_limbs) {
                        bool ok;
                        const uint64_t d = balanced_digits8(gu, ok);
                        if (!ok) atomicOr(a.flags, 1);
#pragma unroll
                        for (int l = 0; l < 8; l++) a.out_limbs[(pr * 8 + l) * a.out_f + row] = (int8_t)(d >> (8 * l));
                    }
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < npairs * 16; idx += blockDim.x) {
                const int p = idx >> 4, r = idx & 15;
                const long long row = (r < 8 ? htA : htB) * 8 + (r & 7);
                if (row < a.out_f && (r < 8 || htB != htA)) {
                    const int64_t y = recombine(red[p][r], a.fw);
                    const long long pr = p0 + p;
                    if (MODE == MODE_LINEAR) a.out[pr * a.out_f + row] = y;
                    else {
                        const int64_t term = mul_shift(y, a.gates[pr], a.fa);
                        const long long tok = a.pair_tok ? a.pair_tok[pr] : 0;
                        atomicAdd(reinterpret_cast<unsigned long long *>(a.out + tok * a.out_f + row),
                                  (unsigned long long)term);
                    }
                }
            }
        }
        __syncthreads();
    }
}

template <int QT, int MODE>
cudaError_t launch_t(const SkinnyArgs &a, int n_groups, int max_pairs, cudaStream_t s) {
    const long long n_ht = (a.out_f + 7) >> 3;
    const long long tiles = MODE == MODE_GATEUP ? n_ht : (n_ht + 1) / 2;
    const int warps = (int)(a.n_blocks < MAX_KSPLIT ? a.n_blocks : MAX_KSPLIT);
    dim3 grid((unsigned)tiles, (unsigned)n_groups), block(32 * warps);
    if (max_pairs <= 1) skinny_kernel<QT, MODE, 1><<<grid, block, 0, s>>>(a);
    else if (max_pairs <= 2) skinny_kernel<QT, MODE, 2><<<grid, block, 0, s>>>(a);
    else skinny_kernel<QT, MODE, 4><<<grid, block, 0, s>>>(a);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_skinny(int qtype, int mode, const SkinnyArgs &a, int n_groups, int max_pairs, cudaStream_t s) {
    if (n_groups <= 0 || a.out_f <= 0 || a.n_blocks <= 0) return cudaErrorInvalidValue;
    if (qtype == QT_Q4K) {
        if (mode == MODE_LINEAR) return launch_t<QT_Q4K, MODE_LINEAR>(a, n_groups, max_pairs, s);
        if (mode == MODE_GATEUP) return launch_t<QT_Q4K, MODE_GATEUP>(a, n_groups, max_pairs, s);
        return launch_t<QT_Q4K, MODE_DOWN>(a, n_groups, max_pairs, s);
    }
    if (qtype == QT_Q6K) {
        if (mode == MODE_LINEAR) return launch_t<QT_Q6K, MODE_LINEAR>(a, n_groups, max_pairs, s);
        if (mode == MODE_GATEUP) return launch_t<QT_Q6K, MODE_GATEUP>(a, n_groups, max_pairs, s);
        return launch_t<QT_Q6K, MODE_DOWN>(a, n_groups, max_pairs, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace iie
