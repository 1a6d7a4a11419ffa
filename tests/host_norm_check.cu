// Host-side check of the exact integer helpers of the block norm (csrc/norm.cuh): the same functions the kernels call,
// compiled for the CPU by nvcc and run over boundary and pseudo-random operands.  Prints "ok <cases>" and exits 0, or the
// first failing operand and exits 1.  Built and run by tests/test_norm_helpers_cpu.py.
#include <cstdio>
#include <cstdlib>
#include "norm.cuh"

using namespace iie;

static unsigned long long lcg_state = 0x9E3779B97F4A7C15ULL;
static unsigned long long lcg() { lcg_state = lcg_state * 6364136223846793005ULL + 1442695040888963407ULL; return lcg_state; }

static int fail(const char *what, u128 v) {
    std::printf("FAIL %s hi=%llx lo=%llx\n", what, (unsigned long long)(v >> 64), (unsigned long long)v);
    return 1;
}

static bool root_ok(u128 v) {
    const u128 r = isqrt128(v);
    if (r >> 64) return false;
    return r * r <= v && (r + 1) * (r + 1) > v;           // v < 2^127 here, so (r + 1)^2 cannot wrap
}

int main() {
    long long cases = 0;
    // ---- floor(sqrt(v)): squares and their neighbours on both sides of the 2^104 switch, then random widths -------------
    const unsigned long long ks[] = {1, 2, 3, 65535, 65536, 65537, 1ULL << 26, (1ULL << 31) - 1, 1ULL << 31, (1ULL << 32) - 1,
                                     1ULL << 32, (1ULL << 32) + 1, (1ULL << 40) + 12345, (1ULL << 51) - 1, 1ULL << 51,
                                     (1ULL << 52) - 1, 1ULL << 52, (1ULL << 52) + 1, (1ULL << 60) + 7, (1ULL << 63) - 1};
    for (unsigned long long k : ks)
        for (int d = -2; d <= 2; d++) {
            if (d < 0 && (u128)k * k < (u128)(-d)) continue;
            const u128 v = (u128)k * k + (u128)(long long)d;
            if (!root_ok(v)) return fail("isqrt128 near a square", v);
            cases++;
        }
    for (int bits = 1; bits <= 126; bits++)
        for (int rep = 0; rep < 400; rep++) {
            u128 v = ((u128)lcg() << 64) | lcg();
            v >>= (128 - bits);
            if (!root_ok(v)) return fail("isqrt128 random", v);
            cases++;
        }
    if (isqrt128(0) != 0) return fail("isqrt128(0)", 0);
    // ---- the reciprocal: never above floor((2^64 - 1) / den), at most eight below ------------------------------------------
    for (int bits = 1; bits <= 62; bits++)
        for (int rep = 0; rep < 2000; rep++) {
            unsigned long long den = lcg() >> (64 - bits);
            if (rep == 0) den = 1ULL << (bits - 1);
            if (rep == 1) den = (1ULL << bits) - 1;
            if (den == 0) den = 1;
            const unsigned long long exact = 0xFFFFFFFFFFFFFFFFULL / den, got = recip_below(den);
            if (got > exact || exact - got > 8) return fail("recip_below", den);
            cases++;
        }
    // ---- floor division through that reciprocal: |num| < 2^62, 0 < den < 2^62, both signs, exact multiples too -------------
    for (int nb = 0; nb <= 62; nb++)
        for (int db = 1; db <= 62; db++)
            for (int rep = 0; rep < 40; rep++) {
                unsigned long long den = lcg() >> (64 - db);
                if (den == 0) den = 1;
                long long num = nb ? (long long)(lcg() >> (64 - nb)) : 0;
                if (rep % 4 == 1) num = (long long)((unsigned long long)num / den * den);      // an exact multiple
                if (rep & 1) num = -num;
                i128 q = (i128)num / (i128)den;
                if ((i128)num % (i128)den != 0 && num < 0) q -= 1;
                if ((i128)floor_div_recip(num, den, recip_below(den)) != q) return fail("floor_div_recip", ((u128)(unsigned long long)num << 64) | den);
                cases++;
            }
    std::printf("ok %lld\n", cases);
    return 0;
}
