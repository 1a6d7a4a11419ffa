// One "item" = one 256-column super-block of a 16-row tile (two repacked 8-row units) multiplied
// with the eight limb columns of one activation vector on a warp MMA.  Shared by the single-token
// streaming kernels and the fused routing kernel.
//
// Column order: MMA column c carries limb col_limb(c) = (c >> 1) + 4 * (c & 1).  With at most four
// limbs in use every odd column is zero and HALF lets each thread skip those scale multiplies.
//
// Instruction diet (the kernels are issue-bound long before they are HBM-bound):
//   * Q4_K high nibbles stay in place (A = 16*q, still a u8) and the factor 16 is divided out of
//     the int32 block sum, which is exact;
//   * Q6_K codes stay unsigned (A = q in 0..63); the -32 offset becomes one extra MMA per sub-block
//     whose A operand is the byte-replicated int8 sub-block scale (sum_j sc_j * sum_i x_i), taken
//     off once per block: T = sum_j sc_j * S_j - 32 * M;
//   * scale bytes are pulled out with single PRMTs; with FAST the block scales are converted with
//     half -> float -> int (exact: an 11-bit significand times a power of two) and kept in 32 bits.
// Bounds: Q4_K |T_lo| < 2^25, |T_hi| = 16 * that < 2^29, min term < 2^21; Q6_K |T| <= 16*128*16*63*128
// < 2^28.3, |32 M| <= 32*16*16*128*128 = 2^27.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace iie {

__device__ __forceinline__ int col_limb(int c) { return (c >> 1) + 4 * (c & 1); }

// byte i of w, zero-extended / sign-extended / replicated into all four bytes: one PRMT each
__device__ __forceinline__ int ubyte_at(uint32_t w, int i) { return (int)__byte_perm(w, 0, 0x4440 | i); }
__device__ __forceinline__ int sbyte_at(uint32_t w, int i) {          // selector msb = replicate the byte's sign
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"((uint32_t)(((8 | i) * 0x1110) | i)));
    return (int)r;
}
__device__ __forceinline__ uint32_t byte_rep(uint32_t w, int i) { return __byte_perm(w, 0, 0x1111 * i); }

// B fragments of one item: 16 words.  Q4_K: sub-block j uses words 2j, 2j+1 (columns 32j + 8t .. +7
// of the block); Q6_K: sub-block (h,kq,u) uses word 8h + 2kq + u (columns 128h + 32kq + 16u + 4t .. +3).
// xcol points at this thread's limb plane, at the first column of the block.
template <int QT, bool GLOBAL>
__device__ __forceinline__ void load_bfrag(const int8_t *xcol, int t, uint32_t (&bf)[16]) {
    if (QT == QT_Q4K) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int8_t *p = xcol + 32 * j + 8 * t;
            const uint2 v = GLOBAL ? ldg64(p) : *reinterpret_cast<const uint2 *>(p);
            bf[2 * j] = v.x; bf[2 * j + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int8_t *p = xcol + 128 * (i >> 3) + 32 * ((i >> 1) & 3) + 16 * (i & 1) + 4 * t;
            bf[i] = GLOBAL ? ldg32(p) : *reinterpret_cast<const uint32_t *>(p);
        }
    }
}

__device__ __forceinline__ uint4 ld128(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

// Exact half * 2^fw as int32 for fw >= 24 when the caller guarantees |result| < 2^31.
__device__ __forceinline__ int scale_small(uint32_t h, int fw) {
    const float v = __half2float(__ushort_as_half((unsigned short)h)) * __int_as_float((127 + fw) << 23);
    return __float2int_rn(v);
}

// D(16x8) = A(16x16,u8) * B(16x8,s8), zero accumulator input
__device__ __forceinline__ void mma_u8s8_k16_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(z));
}

// Q4_K: ua -> MMA rows 0..7, ub -> rows 8..15 (repacked units, any address space).
// FAST: fw >= 24 and every block scale below 2^31 at this fw.  acc[i] is the C-fragment element i.
template <bool FAST, bool HALF>
__device__ __forceinline__ void item_q4k(const uint8_t *ua, const uint8_t *ub, int lane, int fw, const uint32_t (&bf)[16],
                                         int64_t (&acc)[4]) {
    const int g = lane >> 2;
    const uint4 qa0 = ld128(ua + lane * 16), qa1 = ld128(ua + 512 + lane * 16);
    const uint4 qb0 = ld128(ub + lane * 16), qb1 = ld128(ub + 512 + lane * 16);
    const uint4 ma = ld128(ua + 1024 + g * 16), mb = ld128(ub + 1024 + g * 16);
    uint32_t scA[2], mnA[2], scB[2], mnB[2];
    q4k_scales(ma.y, ma.z, ma.w, scA[0], scA[1], mnA[0], mnA[1]);
    q4k_scales(mb.y, mb.z, mb.w, scB[0], scB[1], mnB[0], mnB[1]);
    const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
    int Tlo[4] = {0, 0, 0, 0}, Thi[4] = {0, 0, 0, 0}, M4[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 8; j++) {                             // sub-block j: nibble (j & 1) of group j >> 1
        const int G = j >> 1;
        const uint32_t msk = (j & 1) ? 0xf0f0f0f0u : 0x0f0f0f0fu;
        const uint32_t a0 = wa[2 * G] & msk, a2 = wa[2 * G + 1] & msk, a1 = wb[2 * G] & msk, a3 = wb[2 * G + 1] & msk;
        const int sA = ubyte_at(scA[j >> 2], j & 3), sB = ubyte_at(scB[j >> 2], j & 3);
        const uint32_t mA = byte_rep(mnA[j >> 2], j & 3), mB = byte_rep(mnB[j >> 2], j & 3);
        int c[4];
        mma_u8s8_k32_z(c, a0, a1, a2, a3, bf[2 * j], bf[2 * j + 1]);
        mma_u8s8_k32(M4, mA, mB, mA, mB, bf[2 * j], bf[2 * j + 1]);
        if (j & 1) {
            Thi[0] += sA * c[0]; Thi[2] += sB * c[2];
            if (!HALF) { Thi[1] += sA * c[1]; Thi[3] += sB * c[3]; }
        } else {
            Tlo[0] += sA * c[0]; Tlo[2] += sB * c[2];
            if (!HALF) { Tlo[1] += sA * c[1]; Tlo[3] += sB * c[3]; }
        }
    }
    int T4[4];
#pragma unroll
    for (int i = 0; i < 4; i++) T4[i] = Tlo[i] + (Thi[i] >> 4);            // Thi is an exact multiple of 16
    if (FAST) {
        const int dqA = scale_small(ma.x & 0xFFFF, fw), dmA = scale_small(ma.x >> 16, fw);
        const int dqB = scale_small(mb.x & 0xFFFF, fw), dmB = scale_small(mb.x >> 16, fw);
        acc[0] += (int64_t)dqA * T4[0] - (int64_t)dmA * M4[0];
        acc[2] += (int64_t)dqB * T4[2] - (int64_t)dmB * M4[2];
        if (!HALF) {
            acc[1] += (int64_t)dqA * T4[1] - (int64_t)dmA * M4[1];
            acc[3] += (int64_t)dqB * T4[3] - (int64_t)dmB * M4[3];
        }
    } else {
        const int64_t dqA = half_to_fixed(ma.x & 0xFFFF, fw), dmA = half_to_fixed(ma.x >> 16, fw);
        const int64_t dqB = half_to_fixed(mb.x & 0xFFFF, fw), dmB = half_to_fixed(mb.x >> 16, fw);
        acc[0] += dqA * T4[0] - dmA * M4[0];
        acc[2] += dqB * T4[2] - dmB * M4[2];
        if (!HALF) {
            acc[1] += dqA * T4[1] - dmA * M4[1];
            acc[3] += dqB * T4[3] - dmB * M4[3];
        }
    }
}

template <bool FAST, bool HALF>
__device__ __forceinline__ void item_q6k(const uint8_t *ua, const uint8_t *ub, int lane, int fw, const uint32_t (&bf)[16],
                                         int64_t (&acc)[4]) {
    const int g = lane >> 2;
    const uint4 la0 = ld128(ua + lane * 16), la1 = ld128(ua + 512 + lane * 16), ha = ld128(ua + 1024 + lane * 16);
    const uint4 lb0 = ld128(ub + lane * 16), lb1 = ld128(ub + 512 + lane * 16), hb = ld128(ub + 1024 + lane * 16);
    const uint4 sa = ld128(ua + 1536 + g * 16), sb = ld128(ub + 1536 + g * 16);
    const uint32_t da = *reinterpret_cast<const unsigned short *>(ua + 1664 + g * 2);
    const uint32_t db = *reinterpret_cast<const unsigned short *>(ub + 1664 + g * 2);
    const uint32_t lA[8] = {la0.x, la0.y, la0.z, la0.w, la1.x, la1.y, la1.z, la1.w};   // [h][u]{first 32, second 32}
    const uint32_t lB[8] = {lb0.x, lb0.y, lb0.z, lb0.w, lb1.x, lb1.y, lb1.z, lb1.w};
    const uint32_t hA[4] = {ha.x, ha.y, ha.z, ha.w}, hB[4] = {hb.x, hb.y, hb.z, hb.w};  // [h*2+u]
    const uint32_t sA[4] = {sa.x, sa.y, sa.z, sa.w}, sB[4] = {sb.x, sb.y, sb.z, sb.w};  // 16 int8 scales
    int T4[4] = {0, 0, 0, 0}, M4[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t wAa = lA[(h * 2 + u) * 2], wAb = lA[(h * 2 + u) * 2 + 1], wAh = hA[h * 2 + u];
            const uint32_t wBa = lB[(h * 2 + u) * 2], wBb = lB[(h * 2 + u) * 2 + 1], wBh = hB[h * 2 + u];
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {
                // weight 128h + 32kq + 16u + 4t + i: nibble source word, and 2-bit field kq of the high-bit word
                const uint32_t nA = (kq & 1) ? wAb : wAa, nB = (kq & 1) ? wBb : wBa;
                const uint32_t loA = (kq < 2 ? nA : (nA >> 4)) & 0x0f0f0f0fu, loB = (kq < 2 ? nB : (nB >> 4)) & 0x0f0f0f0fu;
                const uint32_t hiA = ((wAh >> (2 * kq)) << 4) & 0x30303030u, hiB = ((wBh >> (2 * kq)) << 4) & 0x30303030u;
                const int si = 8 * h + 2 * kq + u;
                const int scA = sbyte_at(sA[si >> 2], si & 3), scB = sbyte_at(sB[si >> 2], si & 3);
                const uint32_t b = bf[h * 8 + kq * 2 + u];
                int c[4];
                mma_u8s8_k16_z(c, loA | hiA, loB | hiB, b);                       // unsigned codes 0..63
                mma_s8s8_k16(M4, byte_rep(sA[si >> 2], si & 3), byte_rep(sB[si >> 2], si & 3), b);
                T4[0] += scA * c[0]; T4[2] += scB * c[2];
                if (!HALF) { T4[1] += scA * c[1]; T4[3] += scB * c[3]; }
            }
        }
#pragma unroll
    for (int i = 0; i < 4; i++) T4[i] -= 32 * M4[i];                              // the (q - 32) offset, once per block
    if (FAST) {
        const int dqA = scale_small(da, fw), dqB = scale_small(db, fw);
        acc[0] += (int64_t)dqA * T4[0]; acc[2] += (int64_t)dqB * T4[2];
        if (!HALF) { acc[1] += (int64_t)dqA * T4[1]; acc[3] += (int64_t)dqB * T4[3]; }
    } else {
        const int64_t dqA = half_to_fixed(da, fw), dqB = half_to_fixed(db, fw);
        acc[0] += dqA * T4[0]; acc[2] += dqB * T4[2];
        if (!HALF) { acc[1] += dqA * T4[1]; acc[3] += dqB * T4[3]; }
    }
}

// Runtime dispatch on the limb count (warp-uniform).
template <int QT, bool FAST>
__device__ __forceinline__ void run_item(const uint8_t *ua, const uint8_t *ub, int lane, int fw, const uint32_t (&bf)[16],
                                         bool half, int64_t (&acc)[4]) {
    if (QT == QT_Q4K) {
        if (half) item_q4k<FAST, true>(ua, ub, lane, fw, bf, acc);
        else      item_q4k<FAST, false>(ua, ub, lane, fw, bf, acc);
    } else {
        if (half) item_q6k<FAST, true>(ua, ub, lane, fw, bf, acc);
        else      item_q6k<FAST, false>(ua, ub, lane, fw, bf, acc);
    }
}

// Recombine the eight limb columns of one output row (column order as above) and floor-shift.
__device__ __forceinline__ int64_t recombine_cols(const unsigned long long *cols, int fw) {
    i128 v = 0;
#pragma unroll
    for (int l = 7; l >= 0; l--) v = (v << 8) + (i128)(int64_t)cols[2 * (l & 3) + (l >> 2)];
    return (int64_t)(v >> fw);
}

// Number of balanced digits in use in a packed digit word (highest non-zero digit + 1).
__device__ __forceinline__ int digits_used(uint64_t d) { return d == 0 ? 1 : 8 - (__clzll((long long)d) >> 3); }

}  // namespace iie
