// Shared device helpers for the integer MoE kernels (sm_100a).
//
// Numerics contract (north-mini-code/src/nmc/cohere2.py:97-111, qk_codec.py:54-90):
//   activations are int64 at scale 2^fa, weights are int64 at scale 2^fw derived from raw Q4_K/Q6_K
//   blocks, a linear is one floor shift after an exact full-K sum.  Everything here is exact integer
//   arithmetic; no fast-math, no floating point.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace iie {

typedef __int128 i128;
typedef unsigned __int128 u128;

constexpr int QT_Q4K = 0;
constexpr int QT_Q6K = 1;
constexpr int QT_I64 = 2;          // dense int64 rows (norm gains, dense routers)

// Bytes of one repacked 8-row x 256-column tile ("half-tile block"); equal to 8 raw blocks.
constexpr int HTB_Q4K = 8 * 144;   // 1152
constexpr int HTB_Q6K = 8 * 210;   // 1680

__host__ __device__ inline int htb_bytes(int qtype) { return qtype == QT_Q4K ? HTB_Q4K : HTB_Q6K; }

// round_half_even(half * 2^frac) with integers only.  Every finite half is m * 2^e with an 11-bit
// m, so the product is a shift; a right shift rounds half to even.  Replaces the double + llrint
// conversion of north-mini-code/tools/nmc_qk_kernel.c:16-39 (same values for all finite halves).
__host__ __device__ inline int64_t half_to_fixed(uint32_t h, int frac) {
    const int ex = (h >> 10) & 0x1F;
    const int64_t m = ex ? ((h & 0x3FF) | 0x400) : (h & 0x3FF);
    const int e = (ex ? ex - 25 : -24) + frac;
    int64_t v;
    if (e >= 0) v = (int64_t)((uint64_t)m << (e > 52 ? 52 : e));      // the only path at frac >= 24
    else {
        int s = -e; if (s > 40) s = 40;
        const int64_t q = m >> s, rem = m & (((int64_t)1 << s) - 1), half = (int64_t)1 << (s - 1);
        v = q + ((rem > half) || (rem == half && (q & 1)));
    }
    return (h & 0x8000) ? -v : v;
}

// half * 2^frac when the caller guarantees frac >= 24 (a pure shift) and the result fits int32.
__device__ __forceinline__ int half_to_fixed_small(uint32_t h, int frac) {
    const int ex = (h >> 10) & 0x1F;
    const int m = ex ? ((h & 0x3FF) | 0x400) : (h & 0x3FF);
    const int v = m << ((ex ? ex - 25 : -24) + frac);
    return (h & 0x8000) ? -v : v;
}

// ---- integer sigmoid / SiLU (north-mini-code/src/nmc/_bonsai/fixedpoint.py:74-96,136-163) ----------
__host__ __device__ __forceinline__ int64_t exp2_neg_fixed(int64_t u, int fa) {
    const int s = 16 - fa;
    uint32_t c0 = 65536, c1 = 45426, c2 = 15743, c3 = 3638;          // all operands below stay under 2^32 for fa <= 29
    if (s >= 0) { c0 >>= s; c1 >>= s; c2 >>= s; c3 >>= s; } else { c0 <<= -s; c1 <<= -s; c2 <<= -s; c3 <<= -s; }
    const int64_t k = u >> fa;
    const uint32_t f = (uint32_t)(u & (((int64_t)1 << fa) - 1));
    const uint32_t f2 = (uint32_t)(((uint64_t)f * f) >> fa), f3 = (uint32_t)(((uint64_t)f2 * f) >> fa);
    int64_t p = (int64_t)c0 - (int64_t)(((uint64_t)c1 * f) >> fa) + (int64_t)(((uint64_t)c2 * f2) >> fa) -
                (int64_t)(((uint64_t)c3 * f3) >> fa);
    if (p < 0) p = 0;
    return p >> (k < 63 ? k : 63);
}

// floor(num / z) for 0 <= num < 2^60, 0 < z < 2^31 from a double estimate with an exact fix-up.
__device__ __forceinline__ uint64_t udiv_small(uint64_t num, uint64_t z) {
    uint64_t q = (uint64_t)((double)num / (double)z);
    int64_t r = (int64_t)(num - q * z);
    while (r < 0) { q--; r += (int64_t)z; }
    while (r >= (int64_t)z) { q++; r -= (int64_t)z; }
    return q;
}

// log2(e) at scale 2^fa and the distance beyond which exp2 underflows to zero (fixedpoint.py:136-146).
__host__ __device__ inline int64_t sigmoid_log2e(int fa) { const int s = 16 - fa; return s >= 0 ? ((int64_t)94548 >> s) : ((int64_t)94548 << -s); }
__host__ __device__ inline int64_t sigmoid_clip(int fa) { return (((int64_t)(fa + 2)) << (2 * fa)) / sigmoid_log2e(fa); }

// floor(num / z) for 0 <= num < 2^60, 0 < z < 2^31 with a quotient below 2^31: two single-precision estimates (the
// second one of the remainder) and an exact fix-up; no double-precision division.
// (The host forms of the three conversions let tests/host_fixed_check.cu run the same function on the CPU; the fix-up makes
// the result independent of how the estimates round.)
__host__ __device__ __forceinline__ uint64_t udiv_small_q31(uint64_t num, uint32_t z) {
#ifdef __CUDA_ARCH__
    const float rz = __frcp_rn((float)z);
    uint32_t q = __float2uint_rz((float)(uint32_t)(num >> 29) * rz * 536870912.0f);            // within 2^-21 relative
#else
    const float rz = 1.0f / (float)z;
    uint32_t q = (uint32_t)((float)(uint32_t)(num >> 29) * rz * 536870912.0f);
#endif
    int64_t r = (int64_t)(num - (uint64_t)q * z);                                               // |r| < 2^41
#ifdef __CUDA_ARCH__
    const int q2 = __float2int_rn((float)(int)(r >> 10) * rz * 1024.0f);
#else
    const int q2 = (int)((float)(int)(r >> 10) * rz * 1024.0f + ((r >> 10) >= 0 ? 0.5f : -0.5f));
#endif
    q += q2; r -= (int64_t)q2 * z;
    while (r < 0) { q--; r += z; }
    while (r >= (int64_t)z) { q++; r -= z; }
    return q;
}

// sigmoid(x) = e1 / (e0 + e1) with e0 = 2^-(max(x,0) log2 e), e1 = 2^-((max(x,0) - x) log2 e), both clipped in the
// exponent (fixedpoint.py:136-163).  One of the two exponents is always zero and its power exactly 2^fa, so only the
// other power is evaluated; x = INT64_MIN wraps exactly as the NumPy oracle's int64 arithmetic does.
__host__ __device__ __forceinline__ int64_t sigmoid_fixed_c(int64_t x, int fa, int64_t log2e, int64_t clip) {
    const bool neg = x < 0;
    int64_t d = neg ? (int64_t)(0ULL - (uint64_t)x) : x;
    if (d > clip) d = clip;
    const int64_t es = exp2_neg_fixed((int64_t)((uint64_t)d * (uint64_t)log2e) >> fa, fa);
    const int64_t one = (int64_t)1 << fa;
    return (int64_t)udiv_small_q31((uint64_t)(neg ? es : one) << fa, (uint32_t)(es + one));   // fa <= 29: es + one <= 2^30
}

__host__ __device__ __forceinline__ int64_t sigmoid_fixed(int64_t x, int fa) {
    return sigmoid_fixed_c(x, fa, sigmoid_log2e(fa), sigmoid_clip(fa));
}

__host__ __device__ __forceinline__ int64_t mul_shift(int64_t a, int64_t b, int sh) {
    return (int64_t)(((i128)a * (i128)b) >> sh);
}

__host__ __device__ __forceinline__ int64_t silu_fixed(int64_t x, int fa) { return mul_shift(x, sigmoid_fixed(x, fa), fa); }

// ---- balanced base-256 digits: x = sum_l d_l * 256^l, d_l in [-128,127] --------------------------------
// Eight digits cover |x| <= 127*(2^64-1)/255; `ok` is cleared when a ninth digit would be needed
// (capacity rule of north-mini-code/src/nmc/qk_cuda.py:973-992).
__host__ __device__ __forceinline__ uint64_t balanced_digits8(int64_t x, bool &ok) {
    // with u_l = d_l + 128 in [0, 255]: x + 0x80..80 = sum_l u_l 256^l, so the digits are the bytes of that sum with the
    // top bit flipped.  Every negative int64 has eight digits (the smallest eight-digit number is below INT64_MIN); a
    // positive one does while the sum stays below 2^64.
    constexpr uint64_t C = 0x8080808080808080ULL;
    ok = x <= (int64_t)0x7F7F7F7F7F7F7F7FLL;
    return ((uint64_t)x + C) ^ C;
}

// ---- warp-level integer MMA (legacy tensor path; the decode kernels are HBM-bound) ---------------------
// D(16x8,s32) += A(16x32,u8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8,s32) += A(16x16,s8,row) * B(16x8,s8,col)
__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_s8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Variants with a zero accumulator input (one shared zero register instead of four moves per call).
__device__ __forceinline__ void mma_u8s8_k32_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}
__device__ __forceinline__ void mma_s8s8_k16_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(z));
}

__device__ __forceinline__ uint4 ldg128(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ uint2 ldg64(const void *p) { return __ldg(reinterpret_cast<const uint2 *>(p)); }
__device__ __forceinline__ uint32_t ldg32(const void *p) { return __ldg(reinterpret_cast<const uint32_t *>(p)); }

// Streaming (read-once) 128-bit load that does not pollute L1.
__device__ __forceinline__ uint4 ldg128_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Unpack the 12 packed scale bytes of a Q4_K block (three words) into byte-packed 6-bit values:
// sc_lo/mn_lo hold sub-blocks 0..3, sc_hi/mn_hi hold 4..7 (qk_codec.py:28-35).
__device__ __forceinline__ void q4k_scales(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t &sc_lo, uint32_t &sc_hi,
                                           uint32_t &mn_lo, uint32_t &mn_hi) {
    sc_lo = u0 & 0x3f3f3f3fu;
    mn_lo = u1 & 0x3f3f3f3fu;
    sc_hi = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
    mn_hi = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
}

}  // namespace iie
