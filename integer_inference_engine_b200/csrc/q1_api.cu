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
#include "../../include/iie_qk.h"
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

static void q1_release_model_state();

extern "C" void bonsai_q1_free_weights(void) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (q_ready == 0) cudaDeviceSynchronize();
    for (auto &w : q_w) if (w.live && w.units) cudaFree(w.units);
    q_w.clear();
    q_weight_bytes = 0;
    for (auto &b : q_buf) if (b.p) { cudaFree(b.p); b.p = nullptr; b.cap = 0; q_generation++; }
    q1_release_model_state();                      // uploaded gain / table buffers and decode contexts name these weights
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

// ====================================================================================================
// Whole-model entries of the 1-bit decoder (bonsai/tools/bonsai_q1_gpu.cu:2020-2030 buffers, 2475-2597 standalone
// attention, 3517-3657 decode context, 3694-3819 prefill forward; bridge bonsai/src/trinote/infer_int/gpu_native.py:
// 418-595).  Same names, argument lists and return codes; the layers run on this library's kernels: RMSNorm fused with
// the digit planes of the following products, Q1_0 products with the residual added in their epilogue, per-head
// norms, rotate-half RoPE + K/V append + exact attention (the attention entries of include/iie_qk.h, rope mode 2),
// wrapping SwiGLU fused with the digit planes of the down product.  K/V rows are kept as int32: a value that does
// not fit, like any RMSNorm envelope miss, gives the overflow status (4, or 2 for the standalone attention entries)
// on which the reference bridge redoes the call on the host.
// ====================================================================================================
namespace {

struct DevBuf { int64_t *p = nullptr; size_t n = 0; };
std::vector<DevBuf> q_bufs;
bool valid_buf(long long h, size_t at_least) { return h >= 0 && (size_t)h < q_bufs.size() && q_bufs[(size_t)h].p && q_bufs[(size_t)h].n >= at_least; }

struct Q1Stack {
    long long n_layers = 0, H = 0, Hkv = 0, hd = 0, d = 0, dff = 0, frac = 0, inv_sqrt = 0;
    unsigned long long eps = 1;
    std::vector<long long> wq, wk, wv, wo, w1, wu, w2, n1g, n2g, qng, kng;
    long long finalg = -1, out_head = -1, cos_h = -1, sin_h = -1;
};

bool shaped(long long h, long long out_f, long long in_f) {
    return valid(h) && q_w[(size_t)h].out_f == out_f && q_w[(size_t)h].nb * 128 == in_f;
}

// every handle of the stack names a live tensor of the right shape; rope tables cover `positions` rows
bool stack_ok(const Q1Stack &m, long long positions) {
    if (m.n_layers <= 0 || m.H <= 0 || m.Hkv <= 0 || m.hd <= 0 || m.d <= 0 || m.dff <= 0 || m.H % m.Hkv || m.hd % 2 || m.d % 128 ||
        m.dff % 128 || (m.H * m.hd) % 128 || m.frac < 1 || m.frac > 29 || !attn_shape_ok((int)m.H, (int)m.Hkv, (int)m.hd)) return false;
    const long long qd = m.H * m.hd, kd = m.Hkv * m.hd;
    for (long long li = 0; li < m.n_layers; li++) {
        const size_t i = (size_t)li;
        if (!shaped(m.wq[i], qd, m.d) || !shaped(m.wk[i], kd, m.d) || !shaped(m.wv[i], kd, m.d) || !shaped(m.wo[i], m.d, qd) ||
            !shaped(m.w1[i], m.dff, m.d) || !shaped(m.wu[i], m.dff, m.d) || !shaped(m.w2[i], m.d, m.dff) ||
            !valid_buf(m.n1g[i], (size_t)m.d) || !valid_buf(m.n2g[i], (size_t)m.d) || !valid_buf(m.qng[i], (size_t)m.hd) ||
            !valid_buf(m.kng[i], (size_t)m.hd)) return false;
    }
    const size_t table = (size_t)positions * (size_t)(m.hd / 2);
    return valid(m.out_head) && q_w[(size_t)m.out_head].nb * 128 == m.d && valid_buf(m.finalg, (size_t)m.d) &&
           valid_buf(m.cos_h, table) && valid_buf(m.sin_h, table);
}

void fill_stack(Q1Stack &m, const long long *wq, const long long *wk, const long long *wv, const long long *wo, const long long *w1,
                const long long *wu, const long long *w2, const long long *n1g, const long long *n2g, const long long *qng,
                const long long *kng) {
    const size_t n = (size_t)m.n_layers;
    m.wq.assign(wq, wq + n); m.wk.assign(wk, wk + n); m.wv.assign(wv, wv + n); m.wo.assign(wo, wo + n); m.w1.assign(w1, w1 + n);
    m.wu.assign(wu, wu + n); m.w2.assign(w2, w2 + n); m.n1g.assign(n1g, n1g + n); m.n2g.assign(n2g, n2g + n);
    m.qng.assign(qng, qng + n); m.kng.assign(kng, kng + n);
}

// activation rows of `rows` tokens, one allocation
struct Work {
    void *base = nullptr;
    int64_t *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *qn = nullptr, *kn = nullptr, *att = nullptr, *g = nullptr, *u = nullptr;
};
bool alloc_work(Work &w, const Q1Stack &m, long long rows) {
    const size_t qd = (size_t)(m.H * m.hd), kd = (size_t)(m.Hkv * m.hd), T = (size_t)rows;
    const size_t n = T * ((size_t)m.d + 3 * qd + 3 * kd + 2 * (size_t)m.dff);
    if (cudaMalloc(&w.base, n * 8) != cudaSuccess) { cudaGetLastError(); w.base = nullptr; return false; }
    int64_t *p = (int64_t *)w.base;
    w.x = p; p += T * m.d; w.q = p; p += T * qd; w.qn = p; p += T * qd; w.att = p; p += T * qd;
    w.k = p; p += T * kd; w.kn = p; p += T * kd; w.v = p; p += T * kd; w.g = p; p += T * m.dff; w.u = p;
    return true;
}
void free_work(Work &w) { if (w.base) cudaFree(w.base); w = Work(); }

bool product(long long h, const int8_t *planes, const int64_t *totals, long long T, long long frac, int64_t *out, const int64_t *add = nullptr) {
    const Q1Weight &w = q_w[(size_t)h];
    return launch_q1_apply(w.units, w.sc32, w.out_f, w.nb, planes, totals, T, frac, out, q_stream, add) == cudaSuccess;
}

// One layer on T rows of w.x.  attend(q normalised, k normalised, v) runs rotation, cache append and attention into w.att.
template <typename Attend>
bool layer_rows(const Q1Stack &m, long long li, Work &w, long long T, int *flags, Attend attend) {
    const size_t i = (size_t)li;
    const long long qd = m.H * m.hd, kd = m.Hkv * m.hd, widest = std::max({m.d, qd, m.dff});
    int8_t *planes = (int8_t *)q_ensure(QR_PLANES, (size_t)T * 8 * (size_t)widest);
    int64_t *totals = (int64_t *)q_ensure(QR_TOTALS, (size_t)T * (size_t)(widest / 128) * 8);
    if (!planes || !totals) return false;
    const int f = (int)m.frac;
    bool ok = launch_rmsnorm_planes(w.x, T, m.d, q_bufs[(size_t)m.n1g[i]].p, f, m.eps, nullptr, planes, totals, flags, q_stream) == cudaSuccess &&
              product(m.wq[i], planes, totals, T, m.frac, w.q) && product(m.wk[i], planes, totals, T, m.frac, w.k) &&
              product(m.wv[i], planes, totals, T, m.frac, w.v) &&
              launch_rmsnorm(w.q, T * m.H, m.hd, q_bufs[(size_t)m.qng[i]].p, f, m.eps, w.qn, flags, q_stream) == cudaSuccess &&
              launch_rmsnorm(w.k, T * m.Hkv, m.hd, q_bufs[(size_t)m.kng[i]].p, f, m.eps, w.kn, flags, q_stream) == cudaSuccess;
    ok = ok && attend(w.qn, w.kn, w.v, w.att);
    ok = ok && launch_q1_prep(w.att, T, qd / 128, planes, totals, nullptr, q_stream) == cudaSuccess &&
         product(m.wo[i], planes, totals, T, m.frac, w.x, w.x) &&
         launch_rmsnorm_planes(w.x, T, m.d, q_bufs[(size_t)m.n2g[i]].p, f, m.eps, nullptr, planes, totals, flags, q_stream) == cudaSuccess &&
         product(m.w1[i], planes, totals, T, m.frac, w.g) && product(m.wu[i], planes, totals, T, m.frac, w.u) &&
         launch_q1_prep_swiglu(w.g, w.u, m.dff, f, T, m.dff / 128, planes, totals, q_stream) == cudaSuccess &&
         product(m.w2[i], planes, totals, T, m.frac, w.x, w.x);
    (void)kd;
    return ok;
}

// logits of `rows` rows starting at x: final norm, output matrix
bool head_rows(const Q1Stack &m, const int64_t *x, long long rows, int64_t *logits, int *flags) {
    int8_t *planes = (int8_t *)q_ensure(QR_PLANES, (size_t)rows * 8 * (size_t)m.d);
    int64_t *totals = (int64_t *)q_ensure(QR_TOTALS, (size_t)rows * (size_t)(m.d / 128) * 8);
    return planes && totals &&
           launch_rmsnorm_planes(x, rows, m.d, q_bufs[(size_t)m.finalg].p, (int)m.frac, m.eps, nullptr, planes, totals, flags, q_stream) == cudaSuccess &&
           product(m.out_head, planes, totals, rows, m.frac, logits);
}

// int64 host rows -> int32; false when a value does not fit
bool narrow(const long long *src, size_t n, std::vector<int32_t> &dst) {
    dst.resize(n);
    bool fits = true;
    for (size_t i = 0; i < n; i++) {
        fits = fits && src[i] >= INT32_MIN && src[i] <= INT32_MAX;
        dst[i] = (int32_t)src[i];
    }
    return fits;
}

// `rows` rows of `hd` int64 values -> int32 rows of `hp` >= hd values (zero-filled); false when a value does not fit
bool narrow_rows(const long long *src, size_t rows, long long hd, long long hp, std::vector<int32_t> &dst) {
    dst.assign(rows * (size_t)hp, 0);
    bool fits = true;
    for (size_t r = 0; r < rows; r++)
        for (long long e = 0; e < hd; e++) {
            const long long x = src[r * (size_t)hd + (size_t)e];
            fits = fits && x >= INT32_MIN && x <= INT32_MAX;
            dst[r * (size_t)hp + (size_t)e] = (int32_t)x;
        }
    return fits;
}

// smallest head width the attention kernels take that holds `hd` columns (0: none)
long long padded_head_dim(long long hd) {
    for (long long w : {32LL, 64LL, 128LL, 256LL}) if (hd <= w) return w;
    return 0;
}

// Flags other callers left in the shared word are set aside while one of these entries runs and put back afterwards.
struct FlagScope {
    int earlier = 0;
    bool ok = false;
    FlagScope() { earlier = iie_flags_read_clear(q_stream); ok = earlier >= 0; }
    int finish() { const int f = iie_flags_read_clear(q_stream); if (earlier > 0) iie::restore_flag_bits(earlier); return f; }
};

struct DecodeCtx {
    bool alive = false;
    Q1Stack m;
    long long B = 0, cap = 0, vocab = 0;
    int32_t *K = nullptr, *V = nullptr;            // [n_layers][B][Hkv][cap][hd]
    int64_t *logits = nullptr;
    Work w;
    std::vector<char> wide;                        // per sequence: a seeded value did not fit the int32 rows
};
std::vector<DecodeCtx> q_ctx;
bool valid_ctx(long long h) { return h >= 0 && (size_t)h < q_ctx.size() && q_ctx[(size_t)h].alive; }
void free_ctx(DecodeCtx &c) {
    if (c.K) cudaFree(c.K);
    if (c.V) cudaFree(c.V);
    if (c.logits) cudaFree(c.logits);
    free_work(c.w);
    c = DecodeCtx();
}

}  // namespace

extern "C" long long bonsai_buf_upload_i64(const long long *host, long long n) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!host || n <= 0 || !q_init()) return -1;
    DevBuf b;
    if (cudaMalloc(&b.p, (size_t)n * 8) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (cudaMemcpy(b.p, host, (size_t)n * 8, cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); cudaFree(b.p); return -1; }
    b.n = (size_t)n;
    q_bufs.push_back(b);
    return (long long)q_bufs.size() - 1;
}

extern "C" int bonsai_attention_prefill_gpu(const long long *q, const long long *k, const long long *v, long long H, long long Hkv,
                                            long long hd, long long M, long long L, long long start, long long frac,
                                            long long inv_sqrt_fp, long long *out) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    const long long hp = padded_head_dim(hd);          // zero columns change neither a score nor a kept output column
    if (!q || !k || !v || !out || H <= 0 || Hkv <= 0 || hd <= 0 || M <= 0 || L <= 0 || start < 0 || frac < 1 || frac > 29 || H % Hkv ||
        L != start + M || hp == 0 || !attn_shape_ok((int)H, (int)Hkv, (int)hp)) return fail(1, "prefill attention: bad arguments");
    if (!q_init()) return fail(1, "prefill attention: no usable CUDA device");
    // this library's layouts: queries and new K/V rows token-major, the cache [Hkv][L][hp] int32
    const size_t qd = (size_t)(H * hp), kd = (size_t)(Hkv * hp);
    std::vector<int64_t> qt((size_t)M * qd, 0), kt((size_t)M * kd, 0), vt((size_t)M * kd, 0);
    for (long long h = 0; h < H; h++) for (long long t = 0; t < M; t++)
        memcpy(&qt[(size_t)t * qd + (size_t)(h * hp)], q + ((size_t)h * M + t) * hd, (size_t)hd * 8);
    for (long long h = 0; h < Hkv; h++) for (long long t = 0; t < M; t++) {
        memcpy(&kt[(size_t)t * kd + (size_t)(h * hp)], k + ((size_t)h * L + start + t) * hd, (size_t)hd * 8);
        memcpy(&vt[(size_t)t * kd + (size_t)(h * hp)], v + ((size_t)h * L + start + t) * hd, (size_t)hd * 8);
    }
    std::vector<int32_t> kc, vc;
    const bool k_fits = narrow_rows(k, (size_t)Hkv * L, hd, hp, kc), v_fits = narrow_rows(v, (size_t)Hkv * L, hd, hp, vc);
    if (!k_fits || !v_fits) return fail(2, "prefill attention: a K/V value is beyond int32");
    int64_t *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr; int32_t *dkc = nullptr, *dvc = nullptr;
    bool ok = cudaMalloc(&dq, qt.size() * 8) == cudaSuccess && cudaMalloc(&dk, kt.size() * 8) == cudaSuccess &&
              cudaMalloc(&dv, vt.size() * 8) == cudaSuccess && cudaMalloc(&dout, qt.size() * 8) == cudaSuccess &&
              cudaMalloc(&dkc, kc.size() * 4) == cudaSuccess && cudaMalloc(&dvc, vc.size() * 4) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(dq, qt.data(), qt.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dk, kt.data(), kt.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dv, vt.data(), vt.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dkc, kc.data(), kc.size() * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dvc, vc.data(), vc.size() * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    int flags = -1;
    if (ok) {
        FlagScope scope;
        ok = scope.ok && iie_attn_prefill_dev(dq, dk, dv, dkc, dvc, start, M, 0, nullptr, nullptr, 0, (int)H, (int)Hkv, (int)hp, L, (int)frac,
                                              inv_sqrt_fp, dout, q_stream) == 0;
        flags = scope.finish();
        ok = ok && flags >= 0;
    }
    if (ok && flags == 0) {
        ok = cudaMemcpy(qt.data(), dout, qt.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess;
        if (ok) for (long long h = 0; h < H; h++) for (long long t = 0; t < M; t++)
            memcpy(out + ((size_t)h * M + t) * hd, &qt[(size_t)t * qd + (size_t)(h * hp)], (size_t)hd * 8);
    }
    for (void *p : {(void *)dq, (void *)dk, (void *)dv, (void *)dout, (void *)dkc, (void *)dvc}) if (p) cudaFree(p);
    if (!ok) return fail(1, "prefill attention: CUDA failure");
    if (flags) return fail(2, "prefill attention: a value left the exact envelope");
    return 0;
}

extern "C" int bonsai_attention_decode_batched_gpu(const long long *q, const long long *Kc, const long long *Vc, const long long *lengths,
                                                   long long B, long long H, long long Hkv, long long hd, long long cap, long long frac,
                                                   long long inv_sqrt_fp, long long *out) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    const long long hp = padded_head_dim(hd);
    if (!q || !Kc || !Vc || !lengths || !out || B <= 0 || H <= 0 || Hkv <= 0 || hd <= 0 || cap <= 0 || H % Hkv || frac < 1 || frac > 29 ||
        hp == 0 || !attn_shape_ok((int)H, (int)Hkv, (int)hp)) return fail(1, "batched decode attention: bad arguments");
    for (long long b = 0; b < B; b++) if (lengths[b] < 1 || lengths[b] > cap) return fail(1, "batched decode attention: a length is outside 1..cap");
    if (!q_init()) return fail(1, "batched decode attention: no usable CUDA device");
    const size_t qd = (size_t)(H * hp), kd = (size_t)(Hkv * hp), per_src = (size_t)Hkv * cap * hd, per = (size_t)Hkv * cap * hp;
    std::vector<int32_t> kc, vc;
    const bool k_fits = narrow_rows(Kc, (size_t)B * Hkv * cap, hd, hp, kc), v_fits = narrow_rows(Vc, (size_t)B * Hkv * cap, hd, hp, vc);
    if (!k_fits || !v_fits) {
        // padding rows beyond a sequence's length are not attended to: only values inside the lengths count
        bool fits = true;
        for (long long b = 0; b < B && fits; b++) for (long long h = 0; h < Hkv && fits; h++)
            for (size_t i = 0; i < (size_t)lengths[b] * hd; i++) {
                const size_t at = (size_t)b * per_src + (size_t)h * cap * hd + i;
                if (Kc[at] < INT32_MIN || Kc[at] > INT32_MAX || Vc[at] < INT32_MIN || Vc[at] > INT32_MAX) { fits = false; break; }
            }
        if (!fits) return fail(2, "batched decode attention: a K/V value is beyond int32");
    }
    // the newest row of every sequence (position length - 1) is passed as the step's K/V row and rewritten unchanged
    std::vector<int64_t> qp((size_t)B * qd, 0), kn((size_t)B * kd, 0), vn((size_t)B * kd, 0);
    for (long long b = 0; b < B; b++) {
        for (long long h = 0; h < H; h++) memcpy(&qp[(size_t)b * qd + (size_t)(h * hp)], q + ((size_t)b * H + h) * hd, (size_t)hd * 8);
        for (long long h = 0; h < Hkv; h++) {
            const size_t src = (size_t)b * per_src + ((size_t)h * cap + (size_t)(lengths[b] - 1)) * hd;
            memcpy(&kn[(size_t)b * kd + (size_t)(h * hp)], Kc + src, (size_t)hd * 8);
            memcpy(&vn[(size_t)b * kd + (size_t)(h * hp)], Vc + src, (size_t)hd * 8);
        }
    }
    int64_t *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr; int32_t *dkc = nullptr, *dvc = nullptr;
    bool ok = cudaMalloc(&dq, qp.size() * 8) == cudaSuccess && cudaMalloc(&dout, qp.size() * 8) == cudaSuccess &&
              cudaMalloc(&dk, kn.size() * 8) == cudaSuccess && cudaMalloc(&dv, vn.size() * 8) == cudaSuccess &&
              cudaMalloc(&dkc, kc.size() * 4) == cudaSuccess && cudaMalloc(&dvc, vc.size() * 4) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(dq, qp.data(), qp.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dk, kn.data(), kn.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dv, vn.data(), vn.size() * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dkc, kc.data(), kc.size() * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
         cudaMemcpyAsync(dvc, vc.data(), vc.size() * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    int flags = -1;
    if (ok) {
        FlagScope scope;
        ok = scope.ok;
        for (long long b = 0; ok && b < B; b++)
            ok = iie_attn_decode_dev(dq + (size_t)b * qd, dk + (size_t)b * kd, dv + (size_t)b * kd, dkc + (size_t)b * per, dvc + (size_t)b * per,
                                     lengths[b] - 1, nullptr, 0, nullptr, nullptr, 0, (int)H, (int)Hkv, (int)hp, cap, (int)frac, inv_sqrt_fp,
                                     dout + (size_t)b * qd, q_stream) == 0;
        flags = scope.finish();
        ok = ok && flags >= 0;
    }
    if (ok && flags == 0) {
        ok = cudaMemcpy(qp.data(), dout, qp.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess;
        if (ok) for (long long b = 0; b < B; b++) for (long long h = 0; h < H; h++)
            memcpy(out + ((size_t)b * H + h) * hd, &qp[(size_t)b * qd + (size_t)(h * hp)], (size_t)hd * 8);
    }
    for (void *p : {(void *)dq, (void *)dk, (void *)dv, (void *)dout, (void *)dkc, (void *)dvc}) if (p) cudaFree(p);
    if (!ok) return fail(1, "batched decode attention: CUDA failure");
    if (flags) return fail(2, "batched decode attention: a value left the exact envelope");
    return 0;
}

extern "C" int bonsai_prefill_forward_gpu(const long long *x_embed, long long T, long long d, long long n_layers, long long H, long long Hkv,
                                          long long hd, long long dff, long long frac, long long eps, long long inv_sqrt_fp,
                                          const long long *wq, const long long *wk, const long long *wv, const long long *wo,
                                          const long long *w1, const long long *wu, const long long *w2, const long long *n1g,
                                          const long long *n2g, const long long *qng, const long long *kng, long long finalg,
                                          long long out_head, long long cos_h, long long sin_h, long long *out_logits, long long *out_k,
                                          long long *out_v) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!x_embed || !out_logits || T <= 0 || T > (1 << 20) || n_layers <= 0 || eps < 0 || !wq || !wk || !wv || !wo || !w1 || !wu || !w2 || !n1g ||
        !n2g || !qng || !kng) return fail(1, "prefill forward: bad arguments");
    if (!q_init()) return fail(1, "prefill forward: no usable CUDA device");
    Q1Stack m;
    m.n_layers = n_layers; m.H = H; m.Hkv = Hkv; m.hd = hd; m.d = d; m.dff = dff; m.frac = frac; m.eps = (unsigned long long)eps;
    m.inv_sqrt = inv_sqrt_fp; m.finalg = finalg; m.out_head = out_head; m.cos_h = cos_h; m.sin_h = sin_h;
    fill_stack(m, wq, wk, wv, wo, w1, wu, w2, n1g, n2g, qng, kng);
    if (!stack_ok(m, T)) return fail(1, "prefill forward: a handle or a dimension does not fit the model");
    const long long vocab = q_w[(size_t)out_head].out_f;
    const size_t kv_elems = (size_t)Hkv * T * hd;
    Work w;
    int32_t *kc = nullptr, *vc = nullptr; int64_t *logits = nullptr;
    bool ok = alloc_work(w, m, T) && cudaMalloc(&kc, kv_elems * 4) == cudaSuccess && cudaMalloc(&vc, kv_elems * 4) == cudaSuccess &&
              cudaMalloc(&logits, (size_t)vocab * 8) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(w.x, x_embed, (size_t)T * d * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    int flags = -1;
    std::vector<int32_t> rows;
    if (ok) {
        FlagScope scope;
        ok = scope.ok;
        int *fw = iie::shared_flag_word();
        ok = ok && fw;
        const int64_t *cosd = q_bufs[(size_t)cos_h].p, *sind = q_bufs[(size_t)sin_h].p;
        for (long long li = 0; ok && li < n_layers; li++) {
            ok = layer_rows(m, li, w, T, fw, [&](const int64_t *qn, const int64_t *kn, const int64_t *v, int64_t *att) {
                return iie_attn_prefill_dev(qn, kn, v, kc, vc, 0, T, 0, cosd, sind, 2, (int)H, (int)Hkv, (int)hd, T, (int)frac, inv_sqrt_fp, att,
                                            q_stream) == 0;
            });
            if (ok && (out_k || out_v)) {
                // the layer's cache is the export: K after head norm and rotation, V as projected, [Hkv][T][hd]
                rows.resize(kv_elems);
                for (int which = 0; ok && which < 2; which++) {
                    long long *dst = which ? out_v : out_k;
                    if (!dst) continue;
                    ok = cudaMemcpyAsync(rows.data(), which ? vc : kc, kv_elems * 4, cudaMemcpyDeviceToHost, q_stream) == cudaSuccess &&
                         cudaStreamSynchronize(q_stream) == cudaSuccess;
                    if (ok) for (size_t i = 0; i < kv_elems; i++) dst[(size_t)li * kv_elems + i] = rows[i];
                }
            }
        }
        ok = ok && head_rows(m, w.x + (size_t)(T - 1) * d, 1, logits, fw);
        flags = scope.finish();
        ok = ok && flags >= 0;
    }
    if (ok && flags == 0) ok = cudaMemcpy(out_logits, logits, (size_t)vocab * 8, cudaMemcpyDeviceToHost) == cudaSuccess;
    free_work(w);
    for (void *p : {(void *)kc, (void *)vc, (void *)logits}) if (p) cudaFree(p);
    if (!ok) return fail(1, "prefill forward: CUDA failure");
    if (flags) return fail(4, "prefill forward: a value left the exact envelope");
    return 0;
}

extern "C" long long bonsai_decode_ctx_create(long long B, long long n_layers, long long H, long long Hkv, long long hd, long long d,
                                              long long dff, long long cap, long long vocab, long long frac, long long eps,
                                              long long inv_sqrt, const long long *wq, const long long *wk, const long long *wv,
                                              const long long *wo, const long long *w1, const long long *wu, const long long *w2,
                                              const long long *n1g, const long long *n2g, const long long *qng, const long long *kng,
                                              long long finalg, long long out_head, long long cos_h, long long sin_h) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (B <= 0 || B > 4096 || n_layers <= 0 || cap <= 0 || vocab <= 0 || eps < 0 || !wq || !wk || !wv || !wo || !w1 || !wu || !w2 || !n1g || !n2g ||
        !qng || !kng || !q_init()) { fail(1, "decode context: bad arguments"); return -1; }
    DecodeCtx c;
    Q1Stack &m = c.m;
    m.n_layers = n_layers; m.H = H; m.Hkv = Hkv; m.hd = hd; m.d = d; m.dff = dff; m.frac = frac; m.eps = (unsigned long long)eps;
    m.inv_sqrt = inv_sqrt; m.finalg = finalg; m.out_head = out_head; m.cos_h = cos_h; m.sin_h = sin_h;
    fill_stack(m, wq, wk, wv, wo, w1, wu, w2, n1g, n2g, qng, kng);
    if (!stack_ok(m, cap) || q_w[(size_t)out_head].out_f != vocab) { fail(1, "decode context: a handle or a dimension does not fit the model"); return -1; }
    c.B = B; c.cap = cap; c.vocab = vocab; c.wide.assign((size_t)B, 0);
    const size_t kv = (size_t)n_layers * B * Hkv * cap * hd * 4;
    if (cudaMalloc(&c.K, kv) != cudaSuccess || cudaMalloc(&c.V, kv) != cudaSuccess || cudaMemset(c.K, 0, kv) != cudaSuccess ||
        cudaMemset(c.V, 0, kv) != cudaSuccess || cudaMalloc(&c.logits, (size_t)B * vocab * 8) != cudaSuccess || !alloc_work(c.w, m, B)) {
        cudaGetLastError(); free_ctx(c); fail(2, "decode context: out of device memory"); return -1;
    }
    c.alive = true;
    size_t slot = q_ctx.size();
    for (size_t i = 0; i < q_ctx.size(); i++) if (!q_ctx[i].alive) { slot = i; break; }
    if (slot == q_ctx.size()) q_ctx.emplace_back();
    q_ctx[slot] = std::move(c);
    return (long long)slot;
}

extern "C" int bonsai_decode_ctx_seed_seq(long long ctx_h, long long b, const long long *k_src, const long long *v_src, long long Lb) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!valid_ctx(ctx_h)) return fail(1, "decode context: no such context");
    DecodeCtx &c = q_ctx[(size_t)ctx_h];
    if (b < 0 || b >= c.B || Lb < 0 || Lb > c.cap || (Lb > 0 && (!k_src || !v_src))) return fail(1, "decode context: bad sequence or length");
    if (Lb == 0) return 0;
    const Q1Stack &m = c.m;
    const size_t n = (size_t)m.n_layers * m.Hkv * Lb * m.hd;
    std::vector<int32_t> kn, vn;
    const bool fits_k = narrow(k_src, n, kn), fits_v = narrow(v_src, n, vn);
    if (!fits_k || !fits_v) c.wide[(size_t)b] = 1;           // the next step of this context reports the overflow status
    bool ok = true;
    for (long long li = 0; ok && li < m.n_layers; li++) for (long long h = 0; ok && h < m.Hkv; h++) {
        const size_t src = ((size_t)li * m.Hkv + h) * Lb * m.hd, dst = ((((size_t)li * c.B + b) * m.Hkv + h) * c.cap) * m.hd;
        ok = cudaMemcpyAsync(c.K + dst, kn.data() + src, (size_t)Lb * m.hd * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess &&
             cudaMemcpyAsync(c.V + dst, vn.data() + src, (size_t)Lb * m.hd * 4, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    }
    ok = ok && cudaStreamSynchronize(q_stream) == cudaSuccess;
    return ok ? 0 : fail(1, "decode context: CUDA failure");
}

extern "C" int bonsai_decode_step(long long ctx_h, const long long *x_in, const long long *pos, long long *out_logits) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    clear_error();
    if (!valid_ctx(ctx_h) || !x_in || !pos || !out_logits) return fail(1, "decode step: bad arguments");
    DecodeCtx &c = q_ctx[(size_t)ctx_h];
    const Q1Stack &m = c.m;
    for (long long b = 0; b < c.B; b++) if (pos[b] < 0 || pos[b] >= c.cap) return fail(1, "decode step: a position is outside the cache");
    for (char wide : c.wide) if (wide) return fail(4, "decode step: a seeded K/V value is beyond int32");
    const long long qd = m.H * m.hd, kd = m.Hkv * m.hd;
    const size_t per_seq = (size_t)m.Hkv * c.cap * m.hd;
    bool ok = cudaMemcpyAsync(c.w.x, x_in, (size_t)c.B * m.d * 8, cudaMemcpyHostToDevice, q_stream) == cudaSuccess;
    int flags = -1;
    {
        FlagScope scope;
        ok = ok && scope.ok;
        int *fw = iie::shared_flag_word();
        ok = ok && fw;
        const int64_t *cosd = q_bufs[(size_t)m.cos_h].p, *sind = q_bufs[(size_t)m.sin_h].p;
        for (long long li = 0; ok && li < m.n_layers; li++) {
            int32_t *Kl = c.K + (size_t)li * c.B * per_seq, *Vl = c.V + (size_t)li * c.B * per_seq;
            ok = layer_rows(m, li, c.w, c.B, fw, [&](const int64_t *qn, const int64_t *kn, const int64_t *v, int64_t *att) {
                // sequences sit at their own positions: one single-token attention per sequence
                for (long long b = 0; b < c.B; b++)
                    if (iie_attn_decode_dev(qn + (size_t)b * qd, kn + (size_t)b * kd, v + (size_t)b * kd, Kl + (size_t)b * per_seq,
                                            Vl + (size_t)b * per_seq, pos[b], nullptr, 0, cosd, sind, 2, (int)m.H, (int)m.Hkv, (int)m.hd, c.cap,
                                            (int)m.frac, m.inv_sqrt, att + (size_t)b * qd, q_stream) != 0) return false;
                return true;
            });
        }
        ok = ok && head_rows(m, c.w.x, c.B, c.logits, fw);
        flags = scope.finish();
        ok = ok && flags >= 0;
    }
    if (ok && flags == 0) ok = cudaMemcpy(out_logits, c.logits, (size_t)c.B * c.vocab * 8, cudaMemcpyDeviceToHost) == cudaSuccess;
    if (!ok) return fail(1, "decode step: CUDA failure");
    if (flags) return fail(4, "decode step: a value left the exact envelope");
    return 0;
}

extern "C" void bonsai_decode_ctx_free(long long ctx_h) {
    std::lock_guard<std::recursive_mutex> lk(q_mu);
    if (!valid_ctx(ctx_h)) return;
    cudaDeviceSynchronize();
    free_ctx(q_ctx[(size_t)ctx_h]);
}

static void q1_release_model_state() {
    for (auto &c : q_ctx) if (c.alive) free_ctx(c);
    q_ctx.clear();
    for (auto &b : q_bufs) if (b.p) cudaFree(b.p);
    q_bufs.clear();
}
