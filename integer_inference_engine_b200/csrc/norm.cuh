// Exact integer RMSNorm pieces shared by the routing kernel and the whole-step decode kernel
// (arithmetic of north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72).
#pragma once
#include "common.cuh"

namespace iie {

__host__ __device__ __forceinline__ unsigned long long uabs64(int64_t v) { return v < 0 ? (0ULL - (unsigned long long)v) : (unsigned long long)v; }

// floor(sqrt(v)).  Below 2^104 the root is under 2^52, so the double estimate is within a unit or two of it and the
// residual v - r^2 (under 2^55 in size) is exact in the low 64 bits: the fix-up walks r by the residual in 64-bit words
// (the usual case: the mean square of a residual row is far below that bound); beyond it the bitwise root.
__host__ __device__ inline u128 isqrt128(u128 v) {
    if (v < ((u128)1 << 104)) {
        const double dv = (double)(unsigned long long)(v >> 64) * 18446744073709551616.0 + (double)(unsigned long long)v;
        unsigned long long r = (unsigned long long)sqrt(dv);
        long long e = (long long)((unsigned long long)v - r * r);
        while (e < 0) { r--; e += (long long)(2 * r + 1); }                       // v - (r-1)^2 = e + 2(r-1) + 1
        while (e > (long long)(2 * r)) { e -= (long long)(2 * r + 1); r++; }      // (r+1)^2 <= v  <=>  e >= 2r + 1
        return r;
    }
    u128 res = 0, bit = (u128)1 << 126;
    while (bit > v) bit >>= 2;
    while (bit != 0) {
        if (v >= res + bit) { v -= res + bit; res = (res >> 1) + bit; } else res >>= 1;
        bit >>= 2;
    }
    return res;
}

// A reciprocal for floor_div_recip: any value from a few units below floor((2^64 - 1) / den) up to it serves (the
// quotient estimate only starts lower and the correction loop takes an extra step).  In the middle range a double
// quotient minus its error bound replaces the 64-bit division.
__host__ __device__ __forceinline__ unsigned long long recip_below(unsigned long long den) {
    if (den == 0) return 0;
    if (den >= (1ULL << 13) && den < (1ULL << 60))             // 2^64/den <= 2^51: the double quotient is within 1 of it
        return (unsigned long long)(18446744073709551616.0 / (double)den) - 4;
    return 0xFFFFFFFFFFFFFFFFULL / den;
}

// high half of a 64 x 64-bit product (the host form lets tests/host_norm_check.cu run these helpers on the CPU)
__host__ __device__ __forceinline__ unsigned long long mulhi64(unsigned long long a, unsigned long long b) {
#ifdef __CUDA_ARCH__
    return __umul64hi(a, b);
#else
    return (unsigned long long)(((u128)a * b) >> 64);
#endif
}

// floor(num / den) for |num| < 2^62 and 0 < den < 2^62 through a precomputed reciprocal
// inv <= floor((2^64 - 1) / den) and within a few units of it: the estimate is a few units below the quotient at most.
__host__ __device__ __forceinline__ int64_t floor_div_recip(int64_t num, unsigned long long den, unsigned long long inv) {
    const unsigned long long n = uabs64(num);
    unsigned long long q = mulhi64(n, inv), r = n - q * den;
    while (r >= den) { q++; r -= den; }
    return num >= 0 ? (int64_t)q : -(int64_t)q - (r != 0);
}

}  // namespace iie
