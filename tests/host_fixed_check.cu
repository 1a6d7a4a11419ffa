// The fixed-point helpers of the kernels (csrc/common.cuh: power of two, sigmoid, SiLU, the single-precision floor division,
// balanced base-256 digits) compiled for the CPU by nvcc as a small shared library; tests/test_fixed_helpers_cpu.py loads
// it and compares every function with the NumPy checker over boundary and random operands.
#include "common.cuh"

using namespace iie;

extern "C" {
void h_exp2_neg(const int64_t *u, int64_t *y, long long n, int fa) { for (long long i = 0; i < n; i++) y[i] = exp2_neg_fixed(u[i], fa); }
void h_sigmoid(const int64_t *x, int64_t *y, long long n, int fa) { for (long long i = 0; i < n; i++) y[i] = sigmoid_fixed(x[i], fa); }
void h_silu(const int64_t *x, int64_t *y, long long n, int fa) { for (long long i = 0; i < n; i++) y[i] = silu_fixed(x[i], fa); }
void h_udiv(const uint64_t *num, const uint32_t *z, uint64_t *q, long long n) { for (long long i = 0; i < n; i++) q[i] = udiv_small_q31(num[i], z[i]); }
void h_digits8(const int64_t *x, uint64_t *d, uint8_t *ok, long long n) {
    for (long long i = 0; i < n; i++) { bool o; d[i] = balanced_digits8(x[i], o); ok[i] = o ? 1 : 0; }
}
}
