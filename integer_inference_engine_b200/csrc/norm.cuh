// Exact integer RMSNorm pieces shared by the routing kernel and the whole-step decode kernel
// (arithmetic of north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72).
#pragma once
#include "common.cuh"

namespace iie {

__device__ __forceinline__ unsigned long long uabs64(int64_t v) { return v < 0 ? (0ULL - (unsigned long long)v) : (unsigned long long)v; }

__device__ inline u128 isqrt128(u128 v) {
    if (v < ((u128)1 << 62)) {             // common case: exact from a double estimate plus a fix-up
        const unsigned long long x = (unsigned long long)v;
        unsigned long long r = (unsigned long long)sqrt((double)x);
        while (r * r > x) r--;
        while ((r + 1) * (r + 1) <= x) r++;
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

// floor(num / den) for |num| < 2^62 and 0 < den < 2^62 through a precomputed reciprocal
// inv = floor((2^64 - 1) / den): the estimate is at most 2 below the quotient.
__device__ __forceinline__ int64_t floor_div_recip(int64_t num, unsigned long long den, unsigned long long inv) {
    const unsigned long long n = uabs64(num);
    unsigned long long q = __umul64hi(n, inv), r = n - q * den;
    while (r >= den) { q++; r -= den; }
    return num >= 0 ? (int64_t)q : -(int64_t)q - (r != 0);
}

}  // namespace iie
