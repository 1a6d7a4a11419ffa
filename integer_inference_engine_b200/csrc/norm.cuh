// Exact integer RMSNorm pieces shared by the routing kernel and the whole-step decode kernel
// (arithmetic of north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72).
#pragma once
#include "common.cuh"

namespace iie {

__device__ __forceinline__ unsigned long long uabs64(int64_t v) { return v < 0 ? (0ULL - (unsigned long long)v) : (unsigned long long)v; }

// floor(sqrt(v)).  Below 2^104 a double estimate is off by at most a few units and is fixed up with exact 128-bit
// products (the usual case: the mean square of a residual row is far below that); beyond it the bitwise root.
__device__ inline u128 isqrt128(u128 v) {
    if (v < ((u128)1 << 104)) {
        const double dv = (double)(unsigned long long)(v >> 64) * 18446744073709551616.0 + (double)(unsigned long long)v;
        unsigned long long r = (unsigned long long)sqrt(dv);
        for (int it = 0; it < 8 && (u128)r * r > v; it++) r--;
        for (int it = 0; it < 8 && (u128)(r + 1) * (r + 1) <= v; it++) r++;
        if ((u128)r * r <= v && (u128)(r + 1) * (r + 1) > v) return r;
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
