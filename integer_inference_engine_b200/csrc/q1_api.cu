// C-ABI of the Q1_0 dense path (include/iie_q1.h): registry of re-ordered weights, grow-only device
// scratch, host-pointer entries with the reference's names and return codes, and one device-pointer entry.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "../../include/iie_q1.h"
#include "kernels.h"

using namespace iie;

namespace {

struct Q1Weight {
    uint8_t *units = nullptr;
    long long out_f = 0, nb = 0;
    bool sc32 = false;
    bool live = false;
};

std::recursive_mutex q_mu;
std::vector<Q1Weight> q_w;
unsigned long long q_weight_bytes = 0;
cudaStream_t q_stream = nullptr;
int *q_cells = nullptr;                 // device ints: [0] digits in use, [1] rmsnorm flags
int q_ready = -1;

enum QRole { QR_X, QR_PLANES, QR_TOTALS, QR_OUT, QR_GAIN, QR_COUNT };
struct QBuf { void *p = nullptr; size_t cap = 0; };
unsigned long long q_generation = 0;   // changes whenever a scratch buffer is freed: captured graphs hold the old addresses
QBuf q_buf[QR_COUNT];

thread_local int q_err_code = 0;
thread_local char q_err[256] = "ok";

int fail(int code, const char *fmt, ...) {
    q_err_code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(q_err, sizeof(q_err), fmt, ap);
    va_end(ap);
    cudaGetLastError();
    return code;
}
void clear_error() { q_err_code = 0; memcpy(q_err, "ok", 3); }

bool q_init() {
    if (q_ready >= 0) return q_ready == 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 ||
        cudaStreamCreateWithFlags(&q_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&q_cells, 64) != cudaSuccess || cudaMemset(q_cells, 0, 64) != cudaSuccess) {
        cudaGetLastError(); q_ready = 1; return false;
    }
    q_ready = 0;
    return true;
}

void *q_ensure(int role, size_t bytes) {
    QBuf &b = q_buf[role];
    if (b.p && b.cap >= bytes) return b.p;
    if (b.p) { cudaDeviceSynchronize(); cudaFree(b.p); b.p = nullptr; b.cap = 0; q_generation++; }
    const size_t cap = std::max<size_t>(bytes, 256);
    if (cudaMalloc(&b.p, cap) != cudaSuccess) { cudaGetLastError(); b.p = nullptr; return nullptr; }
    b.cap = cap;
    return b.p;
}

bool valid(long long h) { return h >= 0 && (size_t)h < q_w.size() && q_w[(size_t)h].live; }

// upload + re-order; scale_bits is the width of the caller's scale array
long long register_any(const unsigned char *bits, const void *scale, int scale_bits, long long out_f, long long nb, bool keep) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!bits || !scale || out_f <= 0 || nb <= 0) { fail(1, "q1 register: bad arguments"); return -1; }
    if (!q_init()) { fail(2, "q1 register: no usable CUDA device"); return -1; }
    const size_t bsz = (size_t)out_f * nb * 16, ssz = (size_t)out_f * nb * (scale_bits / 8);
    bool sc32 = scale_bits == 32;
    if (!sc32) {
        sc32 = true;
        const long long *s64 = (const long long *)scale;
        for (size_t i = 0; i < (size_t)out_f * nb; i++)
            if (s64[i] > 0x7FFFFFFFLL || s64[i] < -0x80000000LL) { sc32 = false; break; }
    }
    const long long n_tiles = (out_f + 15) / 16;
    const size_t usz = (size_t)n_tiles * nb * q1_unit_bytes(sc32);
    uint8_t *dbits = nullptr, *dscale = nullptr, *units = nullptr;
    bool ok = cudaMalloc(&dbits, bsz) == cudaSuccess && cudaMalloc(&dscale, ssz) == cudaSuccess &&
              cudaMalloc(&units, usz) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(dbits, bits, bsz, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(dscale, scale, ssz, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    ok = ok && launch_q1_repack(dbits, dscale, scale_bits, sc32, out_f, nb, units, q_stream) == cudaSuccess;
    ok = ok && cudaStreamSynchronize(q_stream) == cudaSuccess;
    if (dbits) cudaFree(dbits);
    if (dscale) cudaFree(dscale);
    if (!ok) { if (units) cudaFree(units); fail(2, "q1 register: CUDA failure"); return -1; }
    Q1Weight w;
    w.units = units; w.out_f = out_f; w.nb = nb; w.sc32 = sc32; w.live = true;
    q_w.push_back(w);
    if (keep) q_weight_bytes += bsz + ssz;
    return (long long)q_w.size() - 1;
}

// product of device-resident x with weight w into device out; returns 0 / 2 / 4
int apply_device(const Q1Weight &w, const int64_t *xd, long long T, long long frac, int64_t *outd, int max_digits,
                 cudaStream_t s) {
    const long long K = w.nb * 128;
    int8_t *planes = (int8_t *)q_ensure(QR_PLANES, (size_t)T * 8 * K);
    int64_t *totals = (int64_t *)q_ensure(QR_TOTALS, (size_t)T * w.nb * 8);
    if (!planes || !totals) return 2;
    int *nl = nullptr;
    if (max_digits < 8) {
        nl = q_cells;
        if (cudaMemsetAsync(nl, 0, sizeof(int), s) != cudaSuccess) return 2;
    }
    if (launch_q1_prep(xd, T, w.nb, planes, totals, nl, s) != cudaSuccess) return 2;
    if (nl) {
        int used = 0;
        if (cudaMemcpyAsync(&used, nl, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
            cudaStreamSynchronize(s) != cudaSuccess) return 2;
        if (used > max_digits) return 4;
    }
    if (launch_q1_apply(w.units, w.sc32, w.out_f, w.nb, planes, totals, T, frac, outd, s) != cudaSuccess) return 2;
    return 0;
}

int apply_host(const Q1Weight &w, const long long *x, long long T, long long frac, long long *out, int max_digits) {
    const size_t xsz = (size_t)T * w.nb * 128 * 8, osz = (size_t)T * w.out_f * 8;
    int64_t *xd = (int64_t *)q_ensure(QR_X, xsz), *od = (int64_t *)q_ensure(QR_OUT, osz);
    if (!xd || !od) return 2;
    if (cudaMemcpyAsync(xd, x, xsz, cudaMemcpyHostToDevice, q_stream) != cudaSuccess) return 2;
    const int rc = apply_device(w, xd, T, frac, od, max_digits, q_stream);
    if (rc != 0) { cudaStreamSynchronize(q_stream); return rc; }
    if (cudaMemcpyAsync(out, od, osz, cudaMemcpyDeviceToHost, q_stream) != cudaSuccess ||
        cudaStreamSynchronize(q_stream) != cudaSuccess) return 2;
    return 0;
}

int one_shot(const long long *x, const unsigned char *bits, const long long *scale, long long tokens, long long out_f,
             long long nb, long long frac, long long *out, int max_digits) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!x || !bits || !scale || !out || tokens <= 0 || out_f <= 0 || nb <= 0) return fail(1, "q1 linear: bad arguments");
    const long long h = register_any(bits, scale, 64, out_f, nb, false);
    if (h < 0) return q_err_code == 1 ? 1 : 2;
    int rc = apply_host(q_w[(size_t)h], (const long long *)x, tokens, frac, out, max_digits);
    cudaFree(q_w[(size_t)h].units);
    q_w.pop_back();                                    // the temporary registration was the last entry
    if (rc == 2) return fail(2, "q1 linear: CUDA failure");
    if (rc == 4) return fail(4, "q1 linear: an activation needs more digits than the caller allowed");
    return 0;
}

}  // namespace

extern "C" int bonsai_gpu_abi_version(void) { return 3; }
extern "C" int bonsai_gpu_last_error_code(void) { return q_err_code; }
extern "C" const char *bonsai_gpu_last_error(void) { return q_err; }

extern "C" int bonsai_gpu_available(void) {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) cudaGetLastError();
    return (e == cudaSuccess && n > 0) ? 0 : 1;
}

extern "C" int bonsai_gpu_mem_info(unsigned long long *free_bytes, unsigned long long *total_bytes) {
    if (!free_bytes || !total_bytes) return 1;
    size_t f = 0, t = 0;
    if (cudaFree(0) != cudaSuccess || cudaMemGetInfo(&f, &t) != cudaSuccess) { cudaGetLastError(); return 2; }
    *free_bytes = f; *total_bytes = t;
    return 0;
}

extern "C" unsigned long long bonsai_q1_resident_weight_bytes(void) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    return q_weight_bytes;
}

extern "C" int bonsai_q1_linear_gpu(const long long *x, const unsigned char *bits, const long long *scale, long long tokens,
                                    long long out_f, long long n_blocks, long long frac, long long *out) {
    const int rc = one_shot(x, bits, scale, tokens, out_f, n_blocks, frac, out, 8);
    return rc == 0 ? 0 : 1;                            // the reference reports every failure of this entry as 1
}

extern "C" int bonsai_q1_linear_dp4a_gpu(const long long *x, const unsigned char *bits, const long long *scale,
                                         long long tokens, long long out_f, long long n_blocks, long long frac, int L,
                                         long long *out) {
    const int LL = L < 0 ? -L : L;
    if (LL < 1 || LL > 8) return 1;
    return one_shot(x, bits, scale, tokens, out_f, n_blocks, frac, out, LL);
}

extern "C" long long bonsai_q1_register_weight(const unsigned char *bits, const long long *scale, long long out_f,
                                               long long n_blocks) {
    return register_any(bits, scale, 64, out_f, n_blocks, true);
}
extern "C" long long bonsai_q1_register_weight_i32(const unsigned char *bits, const int *scale, long long out_f,
                                                   long long n_blocks) {
    return register_any(bits, scale, 32, out_f, n_blocks, true);
}
extern "C" long long bonsai_q1_register_weight_i32_gpu_layout(const unsigned char *bits, const int *scale, long long out_f,
                                                              long long n_blocks) {
    return register_any(bits, scale, 32, out_f, n_blocks, true);
}
extern "C" long long bonsai_q1_register_weight_i32_bmma(const unsigned char *bits, const int *scale, long long out_f,
                                                        long long n_blocks) {
    return register_any(bits, scale, 32, out_f, n_blocks, true);
}

extern "C" int bonsai_q1_apply_resident(long long handle, const long long *x, long long tokens, long long frac,
                                        long long *out) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!valid(handle) || !x || !out || tokens <= 0) return fail(1, "q1 apply: bad arguments");
    const int rc = apply_host(q_w[(size_t)handle], x, tokens, frac, out, 8);
    if (rc != 0) { fail(rc, "q1 apply: CUDA failure"); return 1; }
    return 0;
}

extern "C" void bonsai_q1_free_weights(void) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (q_ready == 0) cudaDeviceSynchronize();
    for (auto &w : q_w) if (w.live && w.units) cudaFree(w.units);
    q_w.clear();
    q_weight_bytes = 0;
    for (auto &b : q_buf) if (b.p) { cudaFree(b.p); b.p = nullptr; b.cap = 0; q_generation++; }
}

extern "C" int bonsai_rmsnorm_gpu(const long long *x, long long rows, long long cols, long long frac, long long eps,
                                  const long long *gain, long long *out) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!x || !out || rows < 0 || cols <= 0 || frac < 0 || frac > 62 || eps < 0) return fail(1, "rmsnorm: bad arguments");
    if (rows == 0) return 0;
    if (!q_init()) return fail(1, "rmsnorm: no usable CUDA device");
    const size_t xsz = (size_t)rows * cols * 8;
    int64_t *xd = (int64_t *)q_ensure(QR_X, xsz), *od = (int64_t *)q_ensure(QR_OUT, xsz), *gd = nullptr;
    if (!xd || !od) return fail(1, "rmsnorm: out of device memory");
    if (gain && !(gd = (int64_t *)q_ensure(QR_GAIN, (size_t)cols * 8))) return fail(1, "rmsnorm: out of device memory");
    int *flags = q_cells + 1;
    int f = 0;
    bool ok = cudaMemcpyAsync(xd, x, xsz, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    ok = ok && (!gain || cudaMemcpyAsync(gd, gain, (size_t)cols * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess);
    ok = ok && cudaMemsetAsync(flags, 0, sizeof(int), q_stream) == cudaSuccess;
    ok = ok && launch_rmsnorm(xd, rows, cols, gd, (int)frac, (unsigned long long)eps, od, flags, q_stream) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(&f, flags, sizeof(int), cudaMemcpyDeviceToHost, q_stream) == cudaSuccess;
    ok = ok && cudaStreamSynchronize(q_stream) == cudaSuccess;
    if (!ok) return fail(1, "rmsnorm: CUDA failure");
    if (f) return fail(4, "rmsnorm: a row left the exact envelope");
    if (cudaMemcpy(out, od, xsz, cudaMemcpyDeviceToHost) != cudaSuccess) return fail(1, "rmsnorm: CUDA failure");
    return 0;
}

extern "C" int iie_q1_apply_dev(long long handle, const int64_t *x_dev, long long tokens, long long frac, int64_t *out_dev,
                                void *stream) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!valid(handle) || !x_dev || !out_dev || tokens <= 0) return 1;
    return apply_device(q_w[(size_t)handle], x_dev, tokens, frac, out_dev, 8, (cudaStream_t)stream);
}

extern "C" int iie_q1_apply_fused_dev(long long handle, int mode, const int64_t *x_dev, const int64_t *x2_dev, long long ld,
                                      const int64_t *gain_dev, long long tokens, long long frac, const int64_t *add_dev,
                                      int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!valid(handle) || !x_dev || !out_dev || tokens <= 0 || mode < 0 || mode > 2 || frac < 1 || frac > 29) return 1;
    const Q1Weight &w = q_w[(size_t)handle];
    const long long K = w.nb * 128, T = tokens;
    cudaStream_t s = (cudaStream_t)stream;
    int8_t *planes = (int8_t *)q_ensure(QR_PLANES, (size_t)T * 8 * K);
    int64_t *totals = (int64_t *)q_ensure(QR_TOTALS, (size_t)T * w.nb * 8);
    if (!planes || !totals) return 2;
    cudaError_t e;
    if (mode == 1) {
        int *flags = iie::shared_flag_word();
        if (!flags) return 2;
        e = iie::launch_rmsnorm_planes(x_dev, T, K, gain_dev, (int)frac, 1ULL, nullptr, planes, totals, flags, s);
    } else if (mode == 2) {
        if (!x2_dev || ld < K) return 1;
        e = iie::launch_q1_prep_swiglu(x_dev, x2_dev, ld, (int)frac, T, w.nb, planes, totals, s);
    } else {
        e = iie::launch_q1_prep(x_dev, T, w.nb, planes, totals, nullptr, s);
    }
    if (e != cudaSuccess) return 2;
    return iie::launch_q1_apply(w.units, w.sc32, w.out_f, w.nb, planes, totals, T, frac, out_dev, s, add_dev) == cudaSuccess ? 0 : 2;
}

extern "C" int iie_q1_head_norm_dev(const int64_t *x_dev, long long rows_a, long long rows_b, long long width, const int64_t *gain_a_dev,
                                    const int64_t *gain_b_dev, long long frac, int64_t *out_dev, void *stream) {
    if (!x_dev || !out_dev || rows_a < 0 || rows_b < 0 || rows_a + rows_b <= 0 || width <= 0 || frac < 1 || frac > 29) return 1;
    int *flags = iie::shared_flag_word();
    if (!flags) return 2;
    return iie::launch_rmsnorm_pair(x_dev, rows_a, rows_b, width, gain_a_dev, gain_b_dev, (int)frac, 1ULL, out_dev, flags,
                                    (cudaStream_t)stream) == cudaSuccess ? 0 : 2;
}

extern "C" unsigned long long iie_q1_workspace_generation(void) { return q_generation; }
extern "C" void iie_q1_set_stream(int on) { iie::set_q1_stream(on); }

extern "C" int iie_q1_silu_mul_dev(const int64_t *gate_dev, const int64_t *up_dev, long long n, long long frac, int64_t *out_dev,
                                   void *stream) {
    if (!gate_dev || !up_dev || !out_dev || n <= 0 || frac < 1 || frac > 29) return 1;
    return iie::launch_q1_silu_mul(gate_dev, up_dev, n, (int)frac, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 2;
}

extern "C" int iie_q1_embed_dev(long long handle, const int *row_dev, long long row, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!valid(handle) || !out_dev) return 1;
    const Q1Weight &w = q_w[(size_t)handle];
    if (!row_dev && (row < 0 || row >= w.out_f)) return 1;
    return iie::launch_q1_embed_row(w.units, w.sc32, w.nb, row_dev, row, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 2;
}

extern "C" int iie_q1_weight_shape(long long handle, long long *out_f, long long *n_blocks, int *scale_bits) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!valid(handle)) return 1;
    const Q1Weight &w = q_w[(size_t)handle];
    if (out_f) *out_f = w.out_f;
    if (n_blocks) *n_blocks = w.nb;
    if (scale_bits) *scale_bits = w.sc32 ? 32 : 64;
    return 0;
}
