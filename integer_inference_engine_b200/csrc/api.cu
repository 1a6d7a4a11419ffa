// C-ABI of the library: weight registry, workspaces, profile counters and the exported entry
// points declared in include/iie_qk.h.  Host pointers cross the boundary in part 1 (the reference's
// ABI v5); part 2 takes device pointers.  No torch types, no exceptions across the boundary.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/iie_qk.h"
#include "kernels.h"
#include "layout.cuh"

using namespace iie;

namespace {

// ---- profile counters (order of north-mini-code/src/nmc/qk_cuda.py:24-34) ----------------------------------
enum Metric {
    PM_REG_CALLS, PM_REG_NS, PM_H2D_CALLS, PM_H2D_BYTES, PM_H2D_NS, PM_D2H_CALLS, PM_D2H_BYTES, PM_D2H_NS,
    PM_ALLOC_CALLS, PM_ALLOC_BYTES, PM_ALLOC_NS, PM_FREE_CALLS, PM_NATIVE_CALLS, PM_RESIDENT_APPLY, PM_GROUPED_APPLY,
    PM_MOE, PM_MOE_BATCHED, PM_MOE_BATCHED_DP4A, PM_Q_CALLS, PM_Q_NS, PM_K_CALLS, PM_K_NS, PM_V_CALLS, PM_V_NS,
    PM_O_CALLS, PM_O_NS, PM_OTHER_CALLS, PM_OTHER_NS, PM_COUNT
};
unsigned long long g_prof[PM_COUNT];
int g_prof_on = 0;
inline void prof(int m, unsigned long long v = 1) { if (g_prof_on) __atomic_fetch_add(&g_prof[m], v, __ATOMIC_RELAXED); }

struct Weight {
    void *d = nullptr;
    long long out_f = 0, nb = 0;       // dense int64: rows, cols
    int qtype = 0;
    size_t bytes = 0;
    unsigned maxd = 0, maxdmin = 0;    // largest |d| / |dmin| half bit patterns
    const uint8_t **cell = nullptr;    // device cell holding `d` (a one-entry pointer table for the kernels)
    bool live = false;
};

struct MoeLayer {
    long long router = -1;
    int n_experts = 0, top_k = 0;
    long long d_model = 0, e_ffn = 0;
    int gate_q = 0, down_q = 0;
    const uint8_t **tabs = nullptr;    // device: [3][n_experts] gate, up, down pointers
    unsigned maxd_gate = 0, maxdmin_gate = 0, maxd_down = 0, maxdmin_down = 0;
    bool live = false;
};

std::recursive_mutex g_mu;
std::vector<Weight> g_w;
std::vector<MoeLayer> g_layers;
cudaStream_t g_stream = nullptr;
int *g_flags = nullptr;               // device flag word
int *g_cells = nullptr;               // device ints: [0] limbs of h, [1] limbs of gate*up, [2] routing ticket
const uint8_t **g_selptr = nullptr;   // device: [3][64] pointers of the experts the last routing selected
int g_pdl = 1;                        // programmatic dependent launch between the decode kernels
long long g_hl_d = 0;                 // width of the digit planes the last single-token routing left in the R_XL scratch
int64_t *g_pow2 = nullptr;            // device: 2^i for i = 0..31 (unit gates at any activation scale)
int g_attn_parity = 0;                // which of the two attention digit-count cells the next block call uses
long long g_tc_min_tokens = 192;      // from this many tokens on, the MoE block runs on the tcgen05 grouped GEMMs
int g_ready = -1;                     // -1 unknown, 0 usable, 1 unusable
int g_stage_mask = 0;                 // profiling: when non-zero, iie_moe_forward_dev runs only these stages
enum Stage { ST_LIMBS = 1, ST_ROUTER = 2, ST_TOPK = 4, ST_GATEUP = 8, ST_DOWN = 16 };
inline bool stage_on(int st) { return g_stage_mask == 0 || (g_stage_mask & st); }

// Persistent device scratch by role, grown on demand (never shrunk until released).
enum Role { R_X, R_XL, R_OUT, R_RAW, R_GU, R_GUL, R_TMP0, R_TMP1, R_TMP2, R_TABS, R_META, R_LOGITS, R_IDS, R_GATES,
            R_GRPOFF, R_PAIRTOK, R_PAIRGATE, R_HNORM, R_ZERO, R_ASCORES, R_AEXP, R_ASTAT, R_APART, R_PSCORES, R_PEXP, R_PSTAT, R_BSCORES, R_BEXP, R_BSTAT, R_BPART, R_XG, R_COUNT };
struct Buf { void *p = nullptr; size_t cap = 0; };
Buf g_buf[R_COUNT];
long long g_ws_allocs = 0;
// Incremented whenever a workspace address a caller may have baked into a captured graph stops being valid (a buffer
// is freed to grow, or the workspaces are released): holders of captured graphs compare it before replaying.
unsigned long long g_ws_generation = 0;

bool init() {
    if (g_ready >= 0) return g_ready == 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); g_ready = 1; return false; }
    if (cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&g_flags, sizeof(int)) != cudaSuccess || cudaMemset(g_flags, 0, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&g_cells, 2048) != cudaSuccess || cudaMemset(g_cells, 0, 2048) != cudaSuccess ||
        cudaMalloc(&g_selptr, 3 * 64 * sizeof(void *)) != cudaSuccess || cudaMalloc(&g_pow2, 32 * sizeof(int64_t)) != cudaSuccess) {
        cudaGetLastError(); g_ready = 1; return false;
    }
    int64_t pw[32];
    for (int i = 0; i < 32; i++) pw[i] = (int64_t)1 << i;
    if (cudaMemcpy(g_pow2, pw, sizeof(pw), cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); g_ready = 1; return false; }
    g_ready = 0;
    return true;
}

void *ensure(int role, size_t bytes) {
    Buf &b = g_buf[role];
    if (b.cap >= bytes && b.p) return b.p;
    if (b.p) { cudaStreamSynchronize(g_stream); cudaFree(b.p); prof(PM_FREE_CALLS); b.p = nullptr; b.cap = 0; g_ws_generation++; }
    size_t cap = std::max<size_t>(bytes, 256);
    if (cudaMalloc(&b.p, cap) != cudaSuccess) { cudaGetLastError(); b.p = nullptr; return nullptr; }
    b.cap = cap; g_ws_allocs++;
    prof(PM_ALLOC_CALLS); prof(PM_ALLOC_BYTES, cap);
    return b.p;
}

void release_workspace() {
    if (g_stream) cudaStreamSynchronize(g_stream);
    for (auto &b : g_buf) if (b.p) { cudaFree(b.p); prof(PM_FREE_CALLS); b.p = nullptr; b.cap = 0; g_ws_generation++; }
}

bool h2d(void *dst, const void *src, size_t n) {
    prof(PM_H2D_CALLS); prof(PM_H2D_BYTES, n);
    return cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, g_stream) == cudaSuccess;
}
bool d2h(void *dst, const void *src, size_t n) {
    prof(PM_D2H_CALLS); prof(PM_D2H_BYTES, n);
    return cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, g_stream) == cudaSuccess;
}
bool sync() { return cudaStreamSynchronize(g_stream) == cudaSuccess; }

bool valid_q(long long h) { return h >= 0 && (size_t)h < g_w.size() && g_w[h].live && g_w[h].qtype != QT_I64; }
bool valid_i64(long long h) { return h >= 0 && (size_t)h < g_w.size() && g_w[h].live && g_w[h].qtype == QT_I64; }

// Fast-path envelope of the streamed kernels (see skinny.cu): the per-limb-column int64 sums
// cannot wrap.  Evaluated with the largest block scales of the tensor at this call's fw.
// Scales small enough for the 32-bit fast conversions of the streaming kernels.
bool small_scales(unsigned maxd, unsigned maxdmin, int fw) {
    if (fw < 24 || fw > 36) return false;
    return half_to_fixed(maxd, fw) < ((int64_t)1 << 31) && half_to_fixed(maxdmin, fw) < ((int64_t)1 << 31);
}

bool fast_envelope(int qtype, long long nb, unsigned maxd, unsigned maxdmin, int fw) {
    if (fw < 0 || fw > 36) return false;
    if ((maxd & 0x7C00u) == 0x7C00u || (maxdmin & 0x7C00u) == 0x7C00u) return false;   // inf/nan scales
    const unsigned __int128 dq = (unsigned __int128)half_to_fixed(maxd, fw), dm = (unsigned __int128)half_to_fixed(maxdmin, fw);
    const unsigned __int128 lim = (unsigned __int128)1 << 62;
    if (qtype == QT_Q4K) return (unsigned __int128)nb * ((dq << 25) + (dm << 21)) < lim;
    return (unsigned __int128)nb * (dq << 28) < lim;
}

int read_flags_clear() {
    int f = 0;
    if (cudaMemcpyAsync(&f, g_flags, sizeof(int), cudaMemcpyDeviceToHost, g_stream) != cudaSuccess) return -1;
    if (cudaMemsetAsync(g_flags, 0, sizeof(int), g_stream) != cudaSuccess) return -1;
    if (!sync()) return -1;
    return f;
}

long long new_slot() {                 // handles are never reused before qk_free_all
    g_w.emplace_back();
    return (long long)g_w.size() - 1;
}

// Upload (or take from device) raw blocks and store them repacked.  Returns handle or -1.
long long register_quant(const void *raw, bool raw_on_device, long long out_f, long long nb, int qtype) {
    if (!init() || !raw || out_f <= 0 || nb <= 0 || (qtype != QT_Q4K && qtype != QT_Q6K)) return -1;
    const int bs = qtype == QT_Q4K ? 144 : 210;
    if (out_f > (1LL << 40) / nb / bs) return -1;
    const size_t raw_bytes = (size_t)out_f * nb * bs;
    const size_t packed = (size_t)((out_f + 7) / 8) * 8 * nb * bs;
    const size_t cell_off = (packed + 255) & ~(size_t)255;
    void *d = nullptr; unsigned *mb = nullptr;
    const uint8_t *src = (const uint8_t *)raw;
    if (cudaMalloc(&d, cell_off + 256) != cudaSuccess) { cudaGetLastError(); return -1; }
    prof(PM_ALLOC_CALLS); prof(PM_ALLOC_BYTES, packed);
    bool ok = true;
    if (!raw_on_device) {
        void *stage = ensure(R_RAW, raw_bytes);
        ok = stage && h2d(stage, raw, raw_bytes);
        src = (const uint8_t *)stage;
    }
    mb = (unsigned *)ensure(R_META, 64);
    unsigned hostmb[2] = {0, 0};
    ok = ok && mb && cudaMemsetAsync(mb, 0, 8, g_stream) == cudaSuccess &&
         cudaMemsetAsync(d, 0, packed, g_stream) == cudaSuccess &&
         launch_repack(src, (uint8_t *)d, out_f, nb, qtype, mb, g_stream) == cudaSuccess &&
         cudaMemcpyAsync((char *)d + cell_off, &d, sizeof(void *), cudaMemcpyHostToDevice, g_stream) == cudaSuccess &&
         cudaMemcpyAsync(hostmb, mb, 8, cudaMemcpyDeviceToHost, g_stream) == cudaSuccess && sync();
    if (!ok) { cudaGetLastError(); cudaFree(d); return -1; }
    const long long h = new_slot();
    Weight &w = g_w[h];
    w.d = d; w.out_f = out_f; w.nb = nb; w.qtype = qtype; w.bytes = packed; w.maxd = hostmb[0]; w.maxdmin = hostmb[1];
    w.cell = (const uint8_t **)((char *)d + cell_off); w.live = true;
    prof(PM_REG_CALLS);
    return h;
}

// y[T,out_f] on device from x[T,K] on device.  check_flags: synchronise and re-run the exact kernel
// if an activation left the limb envelope (host-pointer entries); otherwise flags stay raised.
// Dense product of a prefill-sized batch on the tensor-core tiles; returns false when the shape, the weights or the stream
// (a capture cannot read the digit count back) rule them out, and the caller then takes the batched kernels.
bool linear_tc(const Weight &w, const int8_t *xl, const int *x_nl, long long T, int fw, int64_t *out, cudaStream_t s);

bool linear_dev(const Weight &w, const int64_t *x, long long T, int fw, int64_t *out, bool check_flags, cudaStream_t s,
                const int8_t *xl_ready = nullptr) {
    const long long K = w.nb * 256;
    if (!fast_envelope(w.qtype, w.nb, w.maxd, w.maxdmin, fw))
        return launch_exact_linear((const uint8_t *)w.d, w.qtype, w.out_f, w.nb, x, T, fw, out, s) == cudaSuccess;
    const int8_t *xl = xl_ready;
    const int *x_nl = nullptr;                             // digits in use by the rows, where the planes are made here
    if (!xl) {
        int8_t *buf = (int8_t *)ensure(R_XL, (size_t)T * 8 * K);
        if (!buf) return false;
        if (T >= 2) {
            if (cudaMemsetAsync(g_cells + 4, 0, sizeof(int), s) != cudaSuccess) return false;
            x_nl = g_cells + 4;
        }
        if (launch_limbs(x, T, K, buf, g_flags, s, const_cast<int *>(x_nl)) != cudaSuccess) return false;
        xl = buf;
    }
    if (T >= g_tc_min_tokens && x_nl && g_stage_mask == 0 && linear_tc(w, xl, x_nl, T, fw, out, s)) {
        // done on the tcgen05 tiles
    } else if (T == 1 && w.out_f >= 256 && g_stage_mask == 0) {
        // one row: the bulk-copy streaming kernel (every CTA requests its run of 16-row tiles up front)
        StreamArgs sa = {};
        sa.wa = w.cell; sa.wb = w.cell; sa.n_sel = 1; sa.out_f = w.out_f; sa.n_blocks = w.nb; sa.fw = fw; sa.fa = 16;
        sa.xl = xl; sa.x_per_sel = 0; sa.x_nl = nullptr; sa.out = out; sa.flags = g_flags;
        sa.fast = small_scales(w.maxd, w.maxdmin, fw); sa.pdl = 0;
        if (launch_stream(w.qtype, MODE_LINEAR, sa, s) != cudaSuccess) return false;
    } else if (T >= 2 && T < (1 << 20) && g_stage_mask == 0) {
        // a few rows: one group that owns all of them, every tile streamed once
        int *off = (int *)ensure(R_META, 64);
        if (!off || launch_set2(off, 0, (int)T, s) != cudaSuccess) return false;
        BatchArgs ba = {};
        ba.wa = w.cell; ba.wb = w.cell; ba.grp_off = off; ba.n_groups = 1; ba.out_f = w.out_f; ba.n_blocks = w.nb; ba.fw = fw; ba.fa = 16;
        ba.fast = small_scales(w.maxd, w.maxdmin, fw); ba.xl = xl; ba.x_nl = x_nl; ba.out = out; ba.flags = g_flags;
        if (launch_batch(w.qtype, MODE_LINEAR, ba, s) != cudaSuccess) return false;
    } else {
        SkinnyArgs a = {};
        a.wa = w.cell; a.wb = w.cell; a.pairs_per_group = (int)T; a.out_f = w.out_f; a.n_blocks = w.nb; a.fw = fw; a.fa = 16;
        a.xl = xl; a.out = out; a.flags = g_flags;
        if (launch_skinny(w.qtype, MODE_LINEAR, a, 1, (int)std::min<long long>(T, 4), s) != cudaSuccess) return false;
    }
    if (check_flags) {
        const int f = read_flags_clear();
        if (f < 0) return false;
        if (f & 1) return launch_exact_linear((const uint8_t *)w.d, w.qtype, w.out_f, w.nb, x, T, fw, out, s) == cudaSuccess;
    }
    return true;
}

struct MoePlan {                      // everything the fused MoE kernels need on the device
    const uint8_t *const *gate, *const *up, *const *down;
    int gate_q, down_q;
    long long d_model, e_ffn;
};

// Fused path: limbs(h) -> gate/up (+SiLU*up, limbs of gu) -> down (+gate-weighted accumulate).
// Groups: n_groups experts; grp_expert / grp_off / pair arrays as in SkinnyArgs.  n_pairs activation
// rows of gu are produced.  out [T,d_model] must be initialised by the caller.
bool moe_fused(const MoePlan &p, const int8_t *hl, bool x_bcast_zero, const int *xidx, const int *grp_expert,
               const int *grp_off, int n_groups, long long n_pairs, int max_pairs, const int64_t *pair_gate,
               const int *pair_tok, int fa, int fw, int64_t *out, cudaStream_t s, const int *h_nl = nullptr,
               unsigned maxd_gate = 0x7C00, unsigned maxdmin_gate = 0x7C00, unsigned maxd_down = 0x7C00, unsigned maxdmin_down = 0x7C00) {
    int8_t *gul = (int8_t *)ensure(R_GUL, (size_t)n_pairs * 8 * p.e_ffn);
    if (!gul) return false;
    (void)x_bcast_zero;
    if (!grp_expert && grp_off && g_stage_mask == 0) {
        // groups are the experts themselves: stream every touched expert tile once for all of its rows
        if (cudaMemsetAsync(g_cells + 1, 0, sizeof(int), s) != cudaSuccess) return false;
        BatchArgs ga = {};
        ga.wa = p.gate; ga.wb = p.up; ga.grp_off = grp_off; ga.n_groups = n_groups; ga.out_f = p.e_ffn; ga.n_blocks = p.d_model / 256;
        ga.fw = fw; ga.fa = fa; ga.fast = small_scales(maxd_gate, maxdmin_gate, fw); ga.xl = hl; ga.xidx = xidx; ga.x_nl = h_nl;
        ga.out = nullptr; ga.out_limbs = gul; ga.out_nl = g_cells + 1; ga.flags = g_flags;
        BatchArgs da = {};
        da.wa = p.down; da.wb = p.down; da.grp_off = grp_off; da.n_groups = n_groups; da.out_f = p.d_model; da.n_blocks = p.e_ffn / 256;
        da.fw = fw; da.fa = fa; da.fast = small_scales(maxd_down, maxdmin_down, fw); da.xl = gul; da.xidx = nullptr; da.x_nl = g_cells + 1;
        da.out = out; da.gates = pair_gate; da.pair_tok = pair_tok; da.flags = g_flags;
        const cudaError_t e1 = launch_batch(p.gate_q, MODE_GATEUP, ga, s);
        if (e1 == cudaSuccess) return launch_batch(p.down_q, MODE_DOWN, da, s) == cudaSuccess;
        cudaGetLastError();
        if (e1 != cudaErrorNotSupported) return false;
    }
    SkinnyArgs a = {};
    a.wa = p.gate; a.wb = p.up; a.grp_expert = grp_expert; a.grp_off = grp_off; a.pairs_per_group = 1;
    a.out_f = p.e_ffn; a.n_blocks = p.d_model / 256; a.fw = fw; a.fa = fa; a.xl = hl; a.xidx = xidx;
    a.out = nullptr; a.out_limbs = gul; a.flags = g_flags;
    if (stage_on(ST_GATEUP) && launch_skinny(p.gate_q, MODE_GATEUP, a, n_groups, max_pairs, s) != cudaSuccess) return false;
    SkinnyArgs d = {};
    d.wa = p.down; d.wb = p.down; d.grp_expert = grp_expert; d.grp_off = grp_off; d.pairs_per_group = 1;
    d.out_f = p.d_model; d.n_blocks = p.e_ffn / 256; d.fw = fw; d.fa = fa; d.xl = gul; d.xidx = nullptr;
    d.out = out; d.gates = pair_gate; d.pair_tok = pair_tok; d.flags = g_flags;
    if (!stage_on(ST_DOWN)) return true;
    return launch_skinny(p.down_q, MODE_DOWN, d, n_groups, max_pairs, s) == cudaSuccess;
}

// Unfused exact composition for one (token, expert) pair set; used when the fast envelope fails.
bool moe_exact_pairs(const std::vector<const Weight *> &gw, const std::vector<const Weight *> &uw,
                     const std::vector<const Weight *> &dw, const int64_t *h_dev, const std::vector<int> &pair_tok,
                     const int64_t *gates_dev, long long T, int k, long long d_model, long long e_ffn, int fa, int fw,
                     int64_t *out_dev) {
    const size_t P = gw.size();
    int64_t *g = (int64_t *)ensure(R_TMP0, P * e_ffn * 8), *u = (int64_t *)ensure(R_TMP1, P * e_ffn * 8);
    int64_t *dn = (int64_t *)ensure(R_TMP2, P * d_model * 8);
    if (!g || !u || !dn) return false;
    for (size_t i = 0; i < P; i++) {
        const int64_t *x = h_dev + (size_t)pair_tok[i] * d_model;
        if (launch_exact_linear((const uint8_t *)gw[i]->d, gw[i]->qtype, e_ffn, gw[i]->nb, x, 1, fw, g + i * e_ffn, g_stream) != cudaSuccess ||
            launch_exact_linear((const uint8_t *)uw[i]->d, uw[i]->qtype, e_ffn, uw[i]->nb, x, 1, fw, u + i * e_ffn, g_stream) != cudaSuccess)
            return false;
    }
    if (launch_silu_mul(g, u, (long long)P * e_ffn, fa, g_stream) != cudaSuccess) return false;
    for (size_t i = 0; i < P; i++)
        if (launch_exact_linear((const uint8_t *)dw[i]->d, dw[i]->qtype, d_model, dw[i]->nb, g + i * e_ffn, 1, fw,
                                dn + i * d_model, g_stream) != cudaSuccess) return false;
    return launch_combine(dn, gates_dev, T, k, d_model, fa, out_dev, g_stream) == cudaSuccess;
}

// Largest dequantised |weight| of a tensor family at this fw (from the largest block scales).
unsigned __int128 max_weight(int qtype, unsigned maxd, unsigned maxdmin, int fw) {
    const unsigned __int128 dq = (unsigned __int128)half_to_fixed(maxd, fw), dm = (unsigned __int128)half_to_fixed(maxdmin, fw);
    return qtype == QT_Q4K ? dq * 945 + dm * 63 : dq * 128 * 32;
}
const unsigned __int128 CAP4 = 2139062143ULL;                              // 127 * (256^4 - 1) / 255

int read_cell(int idx, cudaStream_t s) {
    int v = -1;
    if (cudaMemcpyAsync(&v, g_cells + idx, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    return v;
}

bool linear_tc(const Weight &w, const int8_t *xl, const int *x_nl, long long T, int fw, int64_t *out, cudaStream_t s) {
    if (w.qtype != QT_Q4K || w.nb * 256 > 8192 || fw > 32 || !small_scales(w.maxd, w.maxdmin, fw) ||
        max_weight(QT_Q4K, w.maxd, w.maxdmin, fw) > CAP4) return false;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return false; }
    int nl = -1;
    if (cudaMemcpyAsync(&nl, x_nl, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) return false;
    if (nl < 1 || nl > 5) return false;
    int *one_off = (int *)ensure(R_META, 64);
    if (!one_off || launch_set2(one_off, 0, (int)T, s) != cudaSuccess) return false;
    PrefillArgs ra = {};
    ra.wa = w.cell; ra.wb = w.cell; ra.grp_off = one_off; ra.n_experts = 1; ra.n_pairs = T; ra.out_f = w.out_f;
    ra.n_blocks = w.nb; ra.fw = fw; ra.fa = 16; ra.xl = xl; ra.out = out; ra.flags = g_flags;
    if (launch_prefill(QT_Q4K, MODE_LINEAR, nl, ra, s) != cudaSuccess) { cudaGetLastError(); return false; }
    return true;
}

// Expert stage on the tensor-core (tcgen05) tiles for pairs already sorted by group: group x uses the weights
// gate[x] / up[x] / down[x] and owns pairs [off[x], off[x+1]); xidx maps a pair to its row of digit planes, ptok to its
// output row, pg holds its gate weight.  gate/up (+SiLU*up, digit planes of the product) -> down (+gate-weighted combine).
// Returns -1 when the weights or the activation are outside what the tiles carry (the caller then streams), 0 ok, 1 failure.
struct GroupedWeights {
    const uint8_t *const *gate, *const *up, *const *down;
    int gate_q, down_q;
    long long d_model, e_ffn;
    unsigned maxd_gate, maxdmin_gate, maxd_down, maxdmin_down;
};

int grouped_tc(const GroupedWeights &w, int n_groups, const int *off, const int *xidx, const int *ptok, const int64_t *pg,
               const int8_t *hl, int nl_h, long long T, long long P, int fa, int fw, int accumulate, int64_t *out_dev,
               cudaStream_t s) {
    if (w.gate_q != QT_Q4K || w.d_model > 8192 || w.e_ffn > 8192 || nl_h < 1 || nl_h > 4 || fw > 32) return -1;
    if (!small_scales(w.maxd_gate, w.maxdmin_gate, fw) || !small_scales(w.maxd_down, w.maxdmin_down, fw)) return -1;
    if (max_weight(QT_Q4K, w.maxd_gate, w.maxdmin_gate, fw) > CAP4) return -1;
    if (max_weight(w.down_q, w.maxd_down, w.maxdmin_down, fw) > (w.down_q == QT_Q4K ? CAP4 : (unsigned __int128)0x7FFFFFFFULL * 32)) return -1;   // Q6_K: d_q * 128 stays in int32
    int8_t *gul = (int8_t *)ensure(R_GUL, (size_t)P * 8 * w.e_ffn);
    int8_t *xg = xidx ? (int8_t *)ensure(R_XG, (size_t)P * 4 * w.d_model) : nullptr;
    if (!gul || (xidx && !xg)) return 1;
    if (cudaMemsetAsync(g_cells + 1, 0, sizeof(int), s) != cudaSuccess) return 1;
    PrefillArgs ga = {};
    ga.wa = w.gate; ga.wb = w.up; ga.grp_off = off; ga.n_experts = n_groups; ga.n_pairs = P; ga.out_f = w.e_ffn;
    ga.n_blocks = w.d_model / 256; ga.fw = fw; ga.fa = fa; ga.xl = hl; ga.xidx = xidx; ga.xg = xg; ga.out = nullptr; ga.out_limbs = gul;
    ga.out_nl = g_cells + 1; ga.flags = g_flags;
    if (launch_prefill(QT_Q4K, MODE_GATEUP, nl_h, ga, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    const int nl_gu = read_cell(1, s);
    if (nl_gu < 0) return 1;
    if (!accumulate && cudaMemsetAsync(out_dev, 0, (size_t)T * w.d_model * 8, s) != cudaSuccess) return 1;
    PrefillArgs da = {};
    da.wa = w.down; da.wb = w.down; da.grp_off = off; da.n_experts = n_groups; da.n_pairs = P; da.out_f = w.d_model;
    da.n_blocks = w.e_ffn / 256; da.fw = fw; da.fa = fa; da.xl = gul; da.xidx = nullptr; da.out = out_dev; da.gates = pg;
    da.pair_tok = ptok; da.flags = g_flags;
    const cudaError_t de = launch_prefill(w.down_q, MODE_DOWN, nl_gu < 1 ? 1 : nl_gu, da, s);
    if (de == cudaSuccess) return 0;
    cudaGetLastError();
    // the activation needs more digits than the tensor-core tiles carry: streamed kernels for the down stage
    SkinnyArgs d = {};
    d.wa = w.down; d.wb = w.down; d.grp_off = off; d.pairs_per_group = 1; d.out_f = w.d_model; d.n_blocks = w.e_ffn / 256;
    d.fw = fw; d.fa = fa; d.xl = gul; d.out = out_dev; d.gates = pg; d.pair_tok = ptok; d.flags = g_flags;
    return launch_skinny(w.down_q, MODE_DOWN, d, n_groups, 4, s) == cudaSuccess ? 0 : 1;
}

// The same for a registered layer: hl = digit planes of the T hidden rows (nl_h digits in use), ids/gates = routing of
// every row; experts of this layer are ids expert_base .. expert_base + n_experts - 1, other slots are skipped.
int moe_experts_tc(const MoeLayer &L, const int8_t *hl, int nl_h, long long T, const int *ids, const int64_t *gates,
                   int expert_base, int fa, int fw, int accumulate, int64_t *out_dev, cudaStream_t s) {
    const int E = L.n_experts, k = L.top_k;
    const long long P = T * k;
    int *off = (int *)ensure(R_GRPOFF, (size_t)(E + 2) * sizeof(int));
    int *ptok = (int *)ensure(R_PAIRTOK, (size_t)P * sizeof(int));
    int64_t *pg = (int64_t *)ensure(R_PAIRGATE, (size_t)P * 8);
    if (!off || !ptok || !pg) return 1;
    if (launch_dispatch(ids, gates, T, k, E, off, ptok, pg, s, expert_base) != cudaSuccess) return 1;
    const GroupedWeights w = {L.tabs, L.tabs + E, L.tabs + 2 * E, L.gate_q, L.down_q, L.d_model, L.e_ffn,
                              L.maxd_gate, L.maxdmin_gate, L.maxd_down, L.maxdmin_down};
    return grouped_tc(w, E, off, ptok, ptok, pg, hl, nl_h, T, P, fa, fw, accumulate, out_dev, s);
}

// Whole block (router GEMM, top-k, expert stage) on the tensor-core tiles.  Same return codes.
int moe_prefill_tc(const MoeLayer &L, const int64_t *h_dev, long long T, int fa, int fw, int accumulate, int64_t *out_dev,
                   int *ids, int64_t *gates, cudaStream_t s) {
    const Weight &r = g_w[L.router];
    const int E = L.n_experts, k = L.top_k;
    if (r.qtype != QT_Q4K || L.gate_q != QT_Q4K || L.d_model > 8192 || L.e_ffn > 8192) return -1;
    if (!small_scales(r.maxd, r.maxdmin, fw) || max_weight(QT_Q4K, r.maxd, r.maxdmin, fw) > CAP4) return -1;
    int8_t *hl = (int8_t *)ensure(R_XL, (size_t)T * 8 * L.d_model);
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)T * E * 8);
    int *one_off = (int *)ensure(R_META, 64);
    if (!hl || !lg || !one_off) return 1;
    if (cudaMemsetAsync(g_cells, 0, 2 * sizeof(int), s) != cudaSuccess) return 1;
    if (launch_limbs(h_dev, T, L.d_model, hl, g_flags, s, g_cells) != cudaSuccess) return 1;
    const int nl_h = read_cell(0, s);
    if (nl_h < 1 || nl_h > 4) return nl_h < 1 ? 1 : -1;
    // router: one "expert" that owns all T rows
    if (launch_set2(one_off, 0, (int)T, s) != cudaSuccess) return 1;
    PrefillArgs ra = {};
    ra.wa = r.cell; ra.wb = r.cell; ra.grp_off = one_off; ra.n_experts = 1; ra.n_pairs = T; ra.out_f = E;
    ra.n_blocks = L.d_model / 256; ra.fw = fw; ra.fa = fa; ra.xl = hl; ra.out = lg; ra.flags = g_flags;
    if (launch_prefill(QT_Q4K, MODE_LINEAR, nl_h, ra, s) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (launch_topk(lg, T, E, k, fa, ids, gates, s) != cudaSuccess) return 1;
    const int rc = moe_experts_tc(L, hl, nl_h, T, ids, gates, 0, fa, fw, accumulate, out_dev, s);
    if (rc != -1) return rc;
    // routing is done; stream the expert stage
    int *off = (int *)ensure(R_GRPOFF, (size_t)(E + 2) * sizeof(int));
    int *ptok = (int *)ensure(R_PAIRTOK, (size_t)T * k * sizeof(int));
    int64_t *pg = (int64_t *)ensure(R_PAIRGATE, (size_t)T * k * 8);
    if (!off || !ptok || !pg || launch_dispatch(ids, gates, T, k, E, off, ptok, pg, s) != cudaSuccess) return 1;
    if (!accumulate && cudaMemsetAsync(out_dev, 0, (size_t)T * L.d_model * 8, s) != cudaSuccess) return 1;
    MoePlan plan = {L.tabs, L.tabs + E, L.tabs + 2 * E, L.gate_q, L.down_q, L.d_model, L.e_ffn};
    return moe_fused(plan, hl, false, ptok, nullptr, off, E, T * k, (int)std::min<long long>(T, 4), pg, ptok, fa, fw, out_dev, s, g_cells,
                     L.maxd_gate, L.maxdmin_gate, L.maxd_down, L.maxdmin_down) ? 0 : 1;
}

// Single-token fused path: route (optional RMSNorm, limbs, router, top-k) -> gate/up -> down.
// init_mode: 0 leave `out`, 1 zero it, 2 start from x (residual).  Requires a quantised router.
bool moe_decode_token(const MoeLayer &L, const int64_t *x, const int64_t *gain, int fa, int fw, unsigned long long eps,
                      int init_mode, int64_t *out, int *ids, int64_t *gates, cudaStream_t s) {
    const Weight &r = g_w[L.router];
    const int E = L.n_experts, k = L.top_k;
    int8_t *hl = (int8_t *)ensure(R_XL, (size_t)8 * L.d_model);
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)E * 8);
    int8_t *gul = (int8_t *)ensure(R_GUL, (size_t)k * 8 * L.e_ffn);
    if (!hl || !lg || !gul) return false;
    g_hl_d = L.d_model;
    RouteArgs ra = {};
    ra.x = x; ra.gain = gain; ra.d = (int)L.d_model; ra.fa = fa; ra.fw = fw; ra.eps = eps;
    ra.router = (const uint8_t *)r.d; ra.router_q = r.qtype; ra.n_experts = E; ra.k = k;
    ra.hl = hl; ra.h_nl = g_cells; ra.h_out = nullptr; ra.logits = lg; ra.ids = ids; ra.gates = gates;
    ra.init_out = out; ra.init_mode = init_mode; ra.gu_nl = g_cells + 1; ra.counter = (unsigned *)(g_cells + 2);
    ra.flags = g_flags;
    const bool ptrs = k <= 64;
    ra.tabs = ptrs ? L.tabs : nullptr; ra.sel_ptrs = ptrs ? g_selptr : nullptr; ra.pdl = g_pdl;
    if (stage_on(ST_ROUTER) && launch_route(ra, s) != cudaSuccess) return false;
    StreamArgs ga = {};
    ga.wa = L.tabs; ga.wb = L.tabs + E; ga.sel = ids; ga.n_sel = k; ga.out_f = L.e_ffn; ga.n_blocks = L.d_model / 256;
    ga.fw = fw; ga.fa = fa; ga.xl = hl; ga.x_per_sel = 0; ga.x_nl = g_cells; ga.out = nullptr; ga.out_limbs = gul;
    ga.out_nl = g_cells + 1; ga.flags = g_flags; ga.fast = small_scales(L.maxd_gate, L.maxdmin_gate, fw);
    if (ptrs) { ga.sel_wa = g_selptr; ga.sel_wb = g_selptr + k; }
    ga.pdl = g_pdl; ga.early_weights = 0;
    if (stage_on(ST_GATEUP) && launch_stream(L.gate_q, MODE_GATEUP, ga, s) != cudaSuccess) return false;
    StreamArgs da = {};
    da.wa = L.tabs + 2 * E; da.wb = da.wa; da.sel = ids; da.n_sel = k; da.out_f = L.d_model; da.n_blocks = L.e_ffn / 256;
    da.fw = fw; da.fa = fa; da.xl = gul; da.x_per_sel = 1; da.x_nl = g_cells + 1; da.out = out; da.gates = gates;
    da.flags = g_flags; da.fast = small_scales(L.maxd_down, L.maxdmin_down, fw);
    if (ptrs) da.sel_wa = g_selptr + 2 * k;
    // the gate/up kernel releases its dependents only after the routing kernel has completed, so the
    // selected pointers are final when this kernel's CTAs start: its weights may be requested early
    da.pdl = g_pdl; da.early_weights = (g_pdl && ptrs && stage_on(ST_GATEUP)) ? 1 : 0;
    if (stage_on(ST_DOWN) && launch_stream(L.down_q, MODE_DOWN, da, s) != cudaSuccess) return false;
    return true;
}

// Shared implementation of qk_moe_ffn (m = 1, k = n_e) and qk_moe_ffn_batched.
int moe_host_entry(const long long *gate_h, const long long *up_h, const long long *down_h, int m, int k,
                   const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa, int fw,
                   int64_t *out) {
    if (!init() || !gate_h || !up_h || !down_h || !h || !gates || !out || m <= 0 || k <= 0 || d_model <= 0 ||
        e_ffn <= 0 || d_model % 256 || e_ffn % 256 || fa < 1 || fa > 29 || fw < 0 || fw > 62) return 1;
    const size_t P = (size_t)m * k;
    std::vector<const Weight *> gw(P), uw(P), dw(P);
    bool uniform = true;
    for (size_t i = 0; i < P; i++) {
        if (!valid_q(gate_h[i]) || !valid_q(up_h[i]) || !valid_q(down_h[i])) return 1;
        gw[i] = &g_w[gate_h[i]]; uw[i] = &g_w[up_h[i]]; dw[i] = &g_w[down_h[i]];
        if (gw[i]->out_f != e_ffn || uw[i]->out_f != e_ffn || gw[i]->nb != d_model / 256 || uw[i]->nb != d_model / 256 ||
            dw[i]->out_f != d_model || dw[i]->nb != e_ffn / 256) return 1;
        uniform = uniform && gw[i]->qtype == gw[0]->qtype && uw[i]->qtype == gw[0]->qtype && dw[i]->qtype == dw[0]->qtype;
    }
    unsigned mg = 0, mgm = 0, md = 0, mdm = 0;
    for (size_t i = 0; i < P; i++) {
        mg = std::max({mg, gw[i]->maxd, uw[i]->maxd}); mgm = std::max({mgm, gw[i]->maxdmin, uw[i]->maxdmin});
        md = std::max(md, dw[i]->maxd); mdm = std::max(mdm, dw[i]->maxdmin);
    }
    const bool fast = uniform && fast_envelope(gw[0]->qtype, d_model / 256, mg, mgm, fw) &&
                      fast_envelope(dw[0]->qtype, e_ffn / 256, md, mdm, fw);

    int64_t *h_dev = (int64_t *)ensure(R_X, (size_t)m * d_model * 8);
    int64_t *out_dev = (int64_t *)ensure(R_OUT, (size_t)m * d_model * 8);
    int64_t *gates_dev = (int64_t *)ensure(R_GATES, P * 8);
    if (!h_dev || !out_dev || !gates_dev || !h2d(h_dev, h, (size_t)m * d_model * 8) || !h2d(gates_dev, gates, P * 8)) return 1;
    std::vector<int> tok_of(P);
    for (size_t i = 0; i < P; i++) tok_of[i] = (int)(i / k);

    bool done = false;
    if (fast) {
        // group pairs by identical (gate, up, down) triple, in order of first appearance: a table indexed by the gate
        // handle serves the usual case (an expert's three matrices always appear together), an ordered map the rest
        std::vector<std::vector<int>> members;
        {
            std::vector<int> by_gate(g_w.size(), -1);
            bool simple = true;
            for (size_t i = 0; i < P && simple; i++) {
                int &slot = by_gate[(size_t)gate_h[i]];
                if (slot < 0) { slot = (int)members.size(); members.emplace_back(); }
                else { const int f = members[slot][0]; simple = up_h[f] == up_h[i] && down_h[f] == down_h[i]; }
                if (simple) members[slot].push_back((int)i);
            }
            if (!simple) {
                members.clear();
                std::map<std::tuple<long long, long long, long long>, int> index;
                for (size_t i = 0; i < P; i++) {
                    auto key = std::make_tuple(gate_h[i], up_h[i], down_h[i]);
                    auto it = index.find(key);
                    if (it == index.end()) { it = index.emplace(key, (int)members.size()).first; members.emplace_back(); }
                    members[it->second].push_back((int)i);
                }
            }
        }
        const int G = (int)members.size();
        std::vector<const uint8_t *> tabs(3 * (size_t)G);
        std::vector<int> grp_off(G + 1, 0), pair_tok(P);
        std::vector<int64_t> pair_gate(P);
        int maxp = 0, pos = 0;
        for (int gidx = 0; gidx < G; gidx++) {
            const int first = members[gidx][0];
            tabs[gidx] = (const uint8_t *)gw[first]->d; tabs[G + gidx] = (const uint8_t *)uw[first]->d;
            tabs[2 * G + gidx] = (const uint8_t *)dw[first]->d;
            grp_off[gidx] = pos;
            for (int i : members[gidx]) { pair_tok[pos] = tok_of[i]; pair_gate[pos] = gates[i]; pos++; }
            maxp = std::max(maxp, (int)members[gidx].size());
        }
        grp_off[G] = pos;
        const uint8_t **tabs_dev = (const uint8_t **)ensure(R_TABS, std::max<size_t>(tabs.size(), 64) * sizeof(void *));
        int *off_dev = (int *)ensure(R_GRPOFF, (G + 1) * sizeof(int));
        int *tok_dev = (int *)ensure(R_PAIRTOK, P * sizeof(int));
        int64_t *pg_dev = (int64_t *)ensure(R_PAIRGATE, P * 8);
        int8_t *hl = (int8_t *)ensure(R_XL, (size_t)m * 8 * d_model);
        if (!tabs_dev || !off_dev || !tok_dev || !pg_dev || !hl) return 1;
        MoePlan plan = {tabs_dev, tabs_dev + G, tabs_dev + 2 * G, gw[0]->qtype, dw[0]->qtype, d_model, e_ffn};
        bool ok = h2d(tabs_dev, tabs.data(), tabs.size() * sizeof(void *)) && h2d(off_dev, grp_off.data(), (G + 1) * sizeof(int)) &&
                  h2d(tok_dev, pair_tok.data(), P * sizeof(int)) && h2d(pg_dev, pair_gate.data(), P * 8) &&
                  cudaMemsetAsync(out_dev, 0, (size_t)m * d_model * 8, g_stream) == cudaSuccess &&
                  cudaMemsetAsync(g_cells, 0, sizeof(int), g_stream) == cudaSuccess &&
                  launch_limbs(h_dev, m, d_model, hl, g_flags, g_stream, g_cells) == cudaSuccess;
        int tc = -1;
        if (ok && m >= g_tc_min_tokens && g_stage_mask == 0) {
            // prefill-sized call (Engine._moe's batched entry, engine.py:389-411): the grouped tensor-core tiles
            const int nl_h = read_cell(0, g_stream);
            const GroupedWeights w = {tabs_dev, tabs_dev + G, tabs_dev + 2 * G, gw[0]->qtype, dw[0]->qtype, d_model, e_ffn, mg, mgm, md, mdm};
            tc = nl_h < 1 ? 1 : grouped_tc(w, G, off_dev, tok_dev, tok_dev, pg_dev, hl, nl_h, m, (long long)P, fa, fw, 1, out_dev, g_stream);
            ok = tc != 1;
        }
        if (ok && tc < 0)
            ok = moe_fused(plan, hl, false, tok_dev, nullptr, off_dev, G, (long long)P, maxp, pg_dev, tok_dev, fa, fw, out_dev, g_stream,
                           g_cells, mg, mgm, md, mdm);
        if (!ok) { cudaGetLastError(); return 1; }
        const int f = read_flags_clear();
        if (f < 0) return 1;
        done = (f & 1) == 0;                      // an envelope miss re-runs the exact composition below
    }
    if (!done && !moe_exact_pairs(gw, uw, dw, h_dev, tok_of, gates_dev, m, k, d_model, e_ffn, fa, fw, out_dev)) {
        cudaGetLastError(); return 1;
    }
    if (!d2h(out, out_dev, (size_t)m * d_model * 8) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

int apply_resident_impl(long long h, const int64_t *x, long long T, int fw, int64_t *out, int want_qtype) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!init() || !x || !out || T <= 0 || fw < 0 || fw > 62) return 1;
    if (!valid_q(h)) return 1;
    const Weight &w = g_w[h];
    if (want_qtype >= 0 && w.qtype != want_qtype) return 2;
    prof(PM_RESIDENT_APPLY);
    const long long K = w.nb * 256;
    int64_t *xd = (int64_t *)ensure(R_X, (size_t)T * K * 8), *od = (int64_t *)ensure(R_OUT, (size_t)T * w.out_f * 8);
    if (!xd || !od || !h2d(xd, x, (size_t)T * K * 8) || !linear_dev(w, xd, T, fw, od, true, g_stream) ||
        !d2h(out, od, (size_t)T * w.out_f * 8) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

}  // namespace

// ====================================================================================================
// Part 1: reference ABI v5
// ====================================================================================================
namespace iie {
int *shared_flag_word() {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    return init() ? g_flags : nullptr;
}
void restore_flag_bits(int bits) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (bits <= 0 || !init()) return;
    int now = 0;
    if (cudaMemcpy(&now, g_flags, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    now |= bits;
    if (cudaMemcpy(g_flags, &now, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) cudaGetLastError();
}
}  // namespace iie

extern "C" int qk_cuda_abi_version(void) { return 5; }

extern "C" int qk_cuda_available(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    return init() ? 0 : 1;
}

extern "C" void qk_profile_reset(void) { for (auto &v : g_prof) __atomic_store_n(&v, 0ULL, __ATOMIC_RELAXED); }
extern "C" void qk_profile_set_enabled(int enabled) { g_prof_on = enabled ? 1 : 0; }
extern "C" int qk_profile_snapshot(unsigned long long *out, int capacity) {
    if (!out || capacity < PM_COUNT) return -1;
    for (int i = 0; i < PM_COUNT; i++) out[i] = __atomic_load_n(&g_prof[i], __ATOMIC_RELAXED);
    return PM_COUNT;
}

extern "C" int qk_linear_cuda(const uint8_t *W, const int64_t *x, long long T, long long out_f, long long n_blocks,
                              int fw, int qtype, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!W || !x || !out || T <= 0 || fw < 0 || fw > 62) return 1;
    const long long h = register_quant(W, false, out_f, n_blocks, qtype);
    if (h < 0) return 1;
    const int rc = apply_resident_impl(h, x, T, fw, out, -1);
    cudaFree(g_w[h].d); prof(PM_FREE_CALLS);
    g_w.pop_back();                                   // the transient weight is the last slot
    return rc;
}

extern "C" int qk_resident_reserve(long long count) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (count < 0 || count > (1LL << 28)) return 1;
    try { g_w.reserve((size_t)count); } catch (...) { return 1; }
    return 0;
}

extern "C" long long qk_register_weight(const uint8_t *W, long long out_f, long long n_blocks, int qtype) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    return register_quant(W, false, out_f, n_blocks, qtype);
}

extern "C" long long qk_register_i64(const int64_t *W, long long rows, long long cols) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!init() || !W || rows <= 0 || cols <= 0 || rows > (1LL << 40) / cols / 8) return -1;
    void *d = nullptr;
    const size_t bytes = (size_t)rows * cols * 8;
    if (cudaMalloc(&d, bytes) != cudaSuccess) { cudaGetLastError(); return -1; }
    prof(PM_ALLOC_CALLS); prof(PM_ALLOC_BYTES, bytes);
    if (!h2d(d, W, bytes) || !sync()) { cudaGetLastError(); cudaFree(d); return -1; }
    const long long h = new_slot();
    Weight &w = g_w[h];
    w.d = d; w.out_f = rows; w.nb = cols; w.qtype = QT_I64; w.bytes = bytes; w.live = true;
    prof(PM_REG_CALLS);
    return h;
}

extern "C" long long qk_resident_count(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    long long n = 0;
    for (auto &w : g_w) n += w.live ? 1 : 0;
    return n;
}
extern "C" long long qk_resident_capacity(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    return (long long)g_w.capacity();
}

extern "C" void iie_moe_layer_destroy(long long layer);
static void iie_decoders_drop();

extern "C" void qk_free_all(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (g_ready != 0) { std::vector<Weight>().swap(g_w); return; }
    cudaStreamSynchronize(g_stream);
    iie_decoders_drop();
    for (size_t i = 0; i < g_layers.size(); i++) iie_moe_layer_destroy((long long)i);
    g_layers.clear();
    for (auto &w : g_w) if (w.live && w.d) { cudaFree(w.d); prof(PM_FREE_CALLS); }
    std::vector<Weight>().swap(g_w);                  // capacity returns to zero
    release_workspace();
}

extern "C" int qk_apply_resident(long long h, const int64_t *x, long long T, int fw, int64_t *out) {
    return apply_resident_impl(h, x, T, fw, out, -1);
}
extern "C" int qk_apply_resident_q6k_dp4a(long long h, const int64_t *x, long long T, int fw, int Ln, int64_t *out) {
    if (Ln < 1 || Ln > 8) return 1;
    return apply_resident_impl(h, x, T, fw, out, QT_Q6K);
}
extern "C" int qk_apply_resident_q4k_dp4a(long long h, const int64_t *x, long long T, int fw, int Ln, int64_t *out) {
    if (Ln < 1 || Ln > 8) return 1;
    return apply_resident_impl(h, x, T, fw, out, QT_Q4K);
}

extern "C" int qk_apply_resident_grouped(const long long *handles, const int *phase_ids, int count, const int64_t *x,
                                         long long T, int fw, long long output_capacity, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!init() || !handles || !x || !out || count <= 0 || count > 16 || T <= 0 || fw < 0 || fw > 62) return 1;
    long long total = 0, nb = -1;
    for (int i = 0; i < count; i++) {
        if (!valid_q(handles[i])) return 1;
        const Weight &w = g_w[handles[i]];
        if (nb < 0) nb = w.nb; else if (nb != w.nb) return 1;
        total += T * w.out_f;
    }
    if (total > output_capacity) return 1;
    prof(PM_GROUPED_APPLY);
    const long long K = nb * 256;
    int64_t *xd = (int64_t *)ensure(R_X, (size_t)T * K * 8), *od = (int64_t *)ensure(R_OUT, (size_t)total * 8);
    int8_t *xl = (int8_t *)ensure(R_XL, (size_t)T * 8 * K);
    if (!xd || !od || !xl || !h2d(xd, x, (size_t)T * K * 8) ||
        launch_limbs(xd, T, K, xl, g_flags, g_stream) != cudaSuccess) { cudaGetLastError(); return 1; }
    const int f0 = read_flags_clear();
    if (f0 < 0) return 1;
    long long off = 0;
    for (int i = 0; i < count; i++) {
        const Weight &w = g_w[handles[i]];
        const int phase = phase_ids ? phase_ids[i] : 0;
        static const int calls[5] = {PM_OTHER_CALLS, PM_Q_CALLS, PM_K_CALLS, PM_V_CALLS, PM_O_CALLS};
        prof(calls[phase >= 0 && phase <= 4 ? phase : 0]);
        bool ok;
        if (f0 & 1) ok = launch_exact_linear((const uint8_t *)w.d, w.qtype, w.out_f, w.nb, xd, T, fw, od + off, g_stream) == cudaSuccess;
        else ok = linear_dev(w, xd, T, fw, od + off, false, g_stream, xl);
        if (!ok) { cudaGetLastError(); return 1; }
        off += T * w.out_f;
    }
    if (!d2h(out, od, (size_t)total * 8) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int qk_rmsnorm_router(long long gain_h, long long router_h, const int64_t *x, long long rows, int fa, int fw,
                                 unsigned long long eps, int used, long long h_capacity, long long route_capacity,
                                 int64_t *h_out, int *ids_out, int64_t *gates_out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!init() || !x || !h_out || !ids_out || !gates_out || rows <= 0 || used <= 0 || fa < 1 || fa > 29 || fw < 0 ||
        fw > 62 || !valid_i64(gain_h) || !valid_i64(router_h)) return 1;
    const Weight &gain = g_w[gain_h], &router = g_w[router_h];
    const long long width = router.nb, experts = router.out_f;
    if (gain.out_f != 1 || gain.nb != width || used > experts || experts > 1024 || rows * width > h_capacity ||
        rows * used > route_capacity) return 1;
    int64_t *xd = (int64_t *)ensure(R_X, (size_t)rows * width * 8), *hd = (int64_t *)ensure(R_HNORM, (size_t)rows * width * 8);
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)rows * experts * 8), *gd = (int64_t *)ensure(R_GATES, (size_t)rows * used * 8);
    int *idd = (int *)ensure(R_IDS, (size_t)rows * used * sizeof(int));
    if (!xd || !hd || !lg || !gd || !idd || !h2d(xd, x, (size_t)rows * width * 8)) { cudaGetLastError(); return 1; }
    if (launch_rmsnorm(xd, rows, width, (const int64_t *)gain.d, fa, eps, hd, g_flags, g_stream) != cudaSuccess ||
        launch_exact_dense((const int64_t *)router.d, experts, width, hd, rows, fw, lg, g_flags, g_stream) != cudaSuccess ||
        launch_topk(lg, rows, (int)experts, used, fa, idd, gd, g_stream) != cudaSuccess) { cudaGetLastError(); return 1; }
    const int f = read_flags_clear();
    if (f < 0) return 1;
    if (f) return 3;
    if (!d2h(h_out, hd, (size_t)rows * width * 8) || !d2h(ids_out, idd, (size_t)rows * used * sizeof(int)) ||
        !d2h(gates_out, gd, (size_t)rows * used * 8) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int qk_moe_ffn(const long long *gate_h, const long long *up_h, const long long *down_h, int n_e,
                          const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa, int fw,
                          int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS); prof(PM_MOE);
    return moe_host_entry(gate_h, up_h, down_h, 1, n_e, h, gates, d_model, e_ffn, fa, fw, out);
}
extern "C" int qk_moe_ffn_dp4a(const long long *gate_h, const long long *up_h, const long long *down_h, int n_e,
                               const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa,
                               int fw, int64_t *out) {
    return qk_moe_ffn(gate_h, up_h, down_h, n_e, h, gates, d_model, e_ffn, fa, fw, out);
}
extern "C" int qk_moe_ffn_batched(const long long *gate_h, const long long *up_h, const long long *down_h, int m, int k,
                                  const int64_t *h, const int64_t *gates, long long d_model, long long e_ffn, int fa,
                                  int fw, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS); prof(PM_MOE_BATCHED);
    return moe_host_entry(gate_h, up_h, down_h, m, k, h, gates, d_model, e_ffn, fa, fw, out);
}
extern "C" int qk_moe_ffn_batched_dp4a(const long long *gate_h, const long long *up_h, const long long *down_h, int m,
                                       int k, const int64_t *h, const int64_t *gates, long long d_model,
                                       long long e_ffn, int fa, int fw, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS); prof(PM_MOE_BATCHED_DP4A);
    return moe_host_entry(gate_h, up_h, down_h, m, k, h, gates, d_model, e_ffn, fa, fw, out);
}

extern "C" long long qk_moe_workspace_allocations(void) { std::lock_guard<std::recursive_mutex> lk(g_mu); return g_ws_allocs; }
extern "C" unsigned long long qk_moe_workspace_bytes(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    unsigned long long n = 0;
    for (auto &b : g_buf) n += b.cap;
    return n;
}
extern "C" void qk_moe_workspace_release(void) { std::lock_guard<std::recursive_mutex> lk(g_mu); release_workspace(); }

// ====================================================================================================
// Part 2: device-pointer extension
// ====================================================================================================
extern "C" long long iie_register_weight_dev(const void *raw_dev, long long out_f, long long n_blocks, int qtype) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    return register_quant(raw_dev, true, out_f, n_blocks, qtype);
}

extern "C" int iie_weight_export(long long h, void *raw_host) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !raw_host || !valid_q(h)) return 1;
    const Weight &w = g_w[h];
    const size_t raw_bytes = (size_t)w.out_f * w.nb * (w.qtype == QT_Q4K ? 144 : 210);
    void *stage = ensure(R_RAW, raw_bytes);
    if (!stage || launch_unpack((const uint8_t *)w.d, (uint8_t *)stage, w.out_f, w.nb, w.qtype, g_stream) != cudaSuccess ||
        !d2h(raw_host, stage, raw_bytes) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" long long iie_moe_layer_create(long long router_h, const long long *gate_h, const long long *up_h,
                                          const long long *down_h, int n_experts, int top_k, long long d_model,
                                          long long e_ffn) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !gate_h || !up_h || !down_h || n_experts <= 0 || n_experts > 1024 || top_k <= 0 ||
        (router_h >= 0 && top_k > n_experts) ||
        d_model <= 0 || e_ffn <= 0 || d_model % 256 || e_ffn % 256) return -1;
    if (router_h >= 0) {                                // router_h < 0: an expert shard without a router of its own
        if (!(valid_q(router_h) || valid_i64(router_h))) return -1;
        const Weight &r = g_w[router_h];
        if (r.out_f != n_experts || (r.qtype == QT_I64 ? r.nb != d_model : r.nb != d_model / 256)) return -1;
    }
    MoeLayer L;
    std::vector<const uint8_t *> tabs(3 * (size_t)n_experts);
    for (int e = 0; e < n_experts; e++) {
        if (!valid_q(gate_h[e]) || !valid_q(up_h[e]) || !valid_q(down_h[e])) return -1;
        const Weight &g = g_w[gate_h[e]], &u = g_w[up_h[e]], &d = g_w[down_h[e]];
        if (g.out_f != e_ffn || u.out_f != e_ffn || g.nb != d_model / 256 || u.nb != d_model / 256 || d.out_f != d_model ||
            d.nb != e_ffn / 256) return -1;
        if (e == 0) { L.gate_q = g.qtype; L.down_q = d.qtype; }
        if (g.qtype != L.gate_q || u.qtype != L.gate_q || d.qtype != L.down_q) return -1;
        tabs[e] = (const uint8_t *)g.d; tabs[n_experts + e] = (const uint8_t *)u.d; tabs[2 * n_experts + e] = (const uint8_t *)d.d;
        L.maxd_gate = std::max({L.maxd_gate, g.maxd, u.maxd}); L.maxdmin_gate = std::max({L.maxdmin_gate, g.maxdmin, u.maxdmin});
        L.maxd_down = std::max(L.maxd_down, d.maxd); L.maxdmin_down = std::max(L.maxdmin_down, d.maxdmin);
    }
    void *dt = nullptr;
    if (cudaMalloc(&dt, tabs.size() * sizeof(void *)) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (cudaMemcpy(dt, tabs.data(), tabs.size() * sizeof(void *), cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(dt); return -1; }
    L.router = router_h < 0 ? -1 : router_h; L.n_experts = n_experts; L.top_k = top_k; L.d_model = d_model; L.e_ffn = e_ffn;
    L.tabs = (const uint8_t **)dt; L.live = true;
    g_layers.push_back(L);
    return (long long)g_layers.size() - 1;
}

extern "C" void iie_moe_layer_destroy(long long layer) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live) return;
    if (g_stream) cudaStreamSynchronize(g_stream);
    cudaFree((void *)g_layers[layer].tabs);
    g_layers[layer].live = false; g_layers[layer].tabs = nullptr;
}

extern "C" int iie_moe_forward_dev(long long layer, const int64_t *h_dev, long long T, int fa, int fw, int accumulate,
                                   int64_t *out_dev, int *ids_dev, int64_t *gates_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live || !h_dev || !out_dev ||
        T <= 0 || fa < 1 || fa > 29 || g_layers[layer].router < 0) return 1;
    const MoeLayer &L = g_layers[layer];
    const Weight &r = g_w[L.router];
    cudaStream_t s = (cudaStream_t)stream;              // NULL is the CUDA default stream
    if (!fast_envelope(L.gate_q, L.d_model / 256, L.maxd_gate, L.maxdmin_gate, fw) ||
        !fast_envelope(L.down_q, L.e_ffn / 256, L.maxd_down, L.maxdmin_down, fw)) return 3;
    const int E = L.n_experts, k = L.top_k;
    const long long P = T * k;
    if (T == 1 && r.qtype != QT_I64 && L.d_model <= 4096 && k <= 32) {
        int *ids1 = ids_dev ? ids_dev : (int *)ensure(R_IDS, (size_t)P * sizeof(int));
        int64_t *gates1 = gates_dev ? gates_dev : (int64_t *)ensure(R_GATES, (size_t)P * 8);
        if (!ids1 || !gates1) return 1;
        if (!moe_decode_token(L, h_dev, nullptr, fa, fw, 0, accumulate ? 0 : 1, out_dev, ids1, gates1, s)) { cudaGetLastError(); return 1; }
        return 0;
    }
    int *ids = ids_dev ? ids_dev : (int *)ensure(R_IDS, (size_t)P * sizeof(int));
    int64_t *gates = gates_dev ? gates_dev : (int64_t *)ensure(R_GATES, (size_t)P * 8);
    if (!ids || !gates) return 1;
    if (T >= g_tc_min_tokens && g_stage_mask == 0) {
        const int rc = moe_prefill_tc(L, h_dev, T, fa, fw, accumulate, out_dev, ids, gates, s);
        if (rc >= 0) { if (rc) cudaGetLastError(); return rc; }
    }
    int8_t *hl = (int8_t *)ensure(R_XL, (size_t)T * 8 * L.d_model);
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)T * E * 8);
    if (!hl || !lg) return 1;
    if (stage_on(ST_LIMBS) && (cudaMemsetAsync(g_cells, 0, sizeof(int), s) != cudaSuccess ||
                               launch_limbs(h_dev, T, L.d_model, hl, g_flags, s, g_cells) != cudaSuccess)) return 1;
    if (stage_on(ST_ROUTER)) {
        if (r.qtype == QT_I64) {
            if (launch_exact_dense((const int64_t *)r.d, E, L.d_model, h_dev, T, fw, lg, g_flags, s) != cudaSuccess) return 1;
        } else if (!linear_dev(r, h_dev, T, fw, lg, false, s, hl)) return 1;
    }
    if (stage_on(ST_TOPK) && launch_topk(lg, T, E, k, fa, ids, gates, s) != cudaSuccess) return 1;
    if (!accumulate && cudaMemsetAsync(out_dev, 0, (size_t)T * L.d_model * 8, s) != cudaSuccess) return 1;
    MoePlan plan = {L.tabs, L.tabs + E, L.tabs + 2 * E, L.gate_q, L.down_q, L.d_model, L.e_ffn};
    bool ok;
    if (T == 1) {
        // the k selected experts are the groups; every pair reads token 0's limb planes
        const bool fresh = g_buf[R_ZERO].p == nullptr;
        int *zero = (int *)ensure(R_ZERO, 4096 * sizeof(int));          // all-zero index table, written once
        if (!zero || P > 4096) return 1;
        if (fresh && (cudaMemsetAsync(zero, 0, 4096 * sizeof(int), g_stream) != cudaSuccess || !sync())) return 1;
        ok = moe_fused(plan, hl, true, zero, ids, nullptr, k, P, 1, gates, zero, fa, fw, out_dev, s);
    } else {
        int *off = (int *)ensure(R_GRPOFF, (size_t)(E + 1) * sizeof(int));
        int *ptok = (int *)ensure(R_PAIRTOK, (size_t)P * sizeof(int));
        int64_t *pg = (int64_t *)ensure(R_PAIRGATE, (size_t)P * 8);
        if (!off || !ptok || !pg || launch_dispatch(ids, gates, T, k, E, off, ptok, pg, s) != cudaSuccess) return 1;
        ok = moe_fused(plan, hl, false, ptok, nullptr, off, E, P, (int)std::min<long long>(T, 4), pg, ptok, fa, fw, out_dev, s, g_cells,
                       L.maxd_gate, L.maxdmin_gate, L.maxd_down, L.maxdmin_down);
    }
    if (!ok) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int iie_route_dev(long long router_h, int top_k, const int64_t *h_dev, long long T, int fa, int fw,
                             int *ids_dev, int64_t *gates_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !(valid_q(router_h) || valid_i64(router_h)) || !h_dev || !ids_dev || !gates_dev || T <= 0 || fa < 1 ||
        fa > 29) return 1;
    const Weight &r = g_w[router_h];
    const int E = (int)r.out_f;
    const long long d = r.qtype == QT_I64 ? r.nb : r.nb * 256;
    if (top_k <= 0 || top_k > E || E > 1024) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)T * E * 8);
    if (!lg) return 1;
    if (r.qtype == QT_I64) {
        if (launch_exact_dense((const int64_t *)r.d, E, d, h_dev, T, fw, lg, g_flags, s) != cudaSuccess) return 1;
    } else if (!linear_dev(r, h_dev, T, fw, lg, false, s)) { cudaGetLastError(); return 1; }
    return launch_topk(lg, T, E, top_k, fa, ids_dev, gates_dev, s) == cudaSuccess ? 0 : 1;
}

extern "C" int iie_moe_experts_dev(long long layer, const int64_t *h_dev, long long T, const int *ids_dev,
                                   const int64_t *gates_dev, int slots, int expert_base, int fa, int fw, int accumulate,
                                   int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live || !h_dev || !out_dev ||
        !ids_dev || !gates_dev || T <= 0 || slots <= 0 || fa < 1 || fa > 29) return 1;
    MoeLayer L = g_layers[layer];
    L.top_k = slots;                                     // routing slots per row as the caller laid them out
    cudaStream_t s = (cudaStream_t)stream;
    if (!fast_envelope(L.gate_q, L.d_model / 256, L.maxd_gate, L.maxdmin_gate, fw) ||
        !fast_envelope(L.down_q, L.e_ffn / 256, L.maxd_down, L.maxdmin_down, fw)) return 3;
    const int E = L.n_experts;
    const long long P = T * slots;
    int8_t *hl = (int8_t *)ensure(R_XL, (size_t)T * 8 * L.d_model);
    if (!hl) return 1;
    if (cudaMemsetAsync(g_cells, 0, sizeof(int), s) != cudaSuccess) return 1;
    if (launch_limbs(h_dev, T, L.d_model, hl, g_flags, s, g_cells) != cudaSuccess) return 1;
    if (T >= g_tc_min_tokens) {
        const int nl_h = read_cell(0, s);
        if (nl_h < 1) return 1;
        const int rc = moe_experts_tc(L, hl, nl_h, T, ids_dev, gates_dev, expert_base, fa, fw, accumulate, out_dev, s);
        if (rc >= 0) { if (rc) cudaGetLastError(); return rc; }
    }
    int *off = (int *)ensure(R_GRPOFF, (size_t)(E + 2) * sizeof(int));
    int *ptok = (int *)ensure(R_PAIRTOK, (size_t)P * sizeof(int));
    int64_t *pg = (int64_t *)ensure(R_PAIRGATE, (size_t)P * 8);
    if (!off || !ptok || !pg || launch_dispatch(ids_dev, gates_dev, T, slots, E, off, ptok, pg, s, expert_base) != cudaSuccess) return 1;
    if (!accumulate && cudaMemsetAsync(out_dev, 0, (size_t)T * L.d_model * 8, s) != cudaSuccess) return 1;
    MoePlan plan = {L.tabs, L.tabs + E, L.tabs + 2 * E, L.gate_q, L.down_q, L.d_model, L.e_ffn};
    if (!moe_fused(plan, hl, false, ptok, nullptr, off, E, P, (int)std::min<long long>(T, 4), pg, ptok, fa, fw, out_dev, s, g_cells,
                   L.maxd_gate, L.maxdmin_gate, L.maxd_down, L.maxdmin_down)) {
        cudaGetLastError(); return 1;
    }
    return 0;
}

namespace {

// scratch of the attention passes; returns false on allocation failure.  The statistics are reset once per
// (re)allocation or shape change; every call leaves them reset.
bool attn_scratch(AttnArgs &a, cudaStream_t s) {
    static void *last_ptr = nullptr;
    static int last_h = 0, last_hd = 0;
    a.scores = (int64_t *)ensure(R_ASCORES, (size_t)a.H * a.Lmax * 8);
    a.e = (int32_t *)ensure(R_AEXP, (size_t)a.H * a.Lmax * 4);
    uint8_t *st = (uint8_t *)ensure(R_ASTAT, (size_t)a.H * 16 + (size_t)a.H * a.hd * 8 + 2048);     // + the ticket and 256 barrier counters
    // per-chunk partial sums: 64-key chunks, or one chunk per SM of a KV head (at most 192 chunks on any device this targets)
    a.partial = (long long *)ensure(R_APART, (size_t)std::max<long long>((a.Lmax + 63) / 64, 192) * a.H * a.hd * 8);
    if (!a.scores || !a.e || !st || !a.partial) return false;
    a.hmax = (long long *)st; a.Z = (unsigned long long *)(st + (size_t)a.H * 8);
    a.acc = (long long *)(st + (size_t)a.H * 16); a.ticket = (unsigned *)(st + (size_t)a.H * 16 + (size_t)a.H * a.hd * 8);
    if (st != last_ptr || a.H != last_h || a.hd != last_hd) {
        if (launch_attn_reset(a.hmax, a.Z, a.acc, a.ticket, a.H, a.hd, s) != cudaSuccess) return false;
        last_ptr = st; last_h = a.H; last_hd = a.hd;
    }
    return true;
}

void attn_consts(AttnArgs &a, int fa, long long inv_sqrt) {
    a.fa = fa; a.inv_sqrt = inv_sqrt; a.log2e = sigmoid_log2e(fa);
    const long long ca = (((long long)(fa + 2)) << (2 * fa)) / a.log2e, cb = ((long long)1 << 62) / a.log2e;
    a.clip = ca < cb ? ca : cb;
}

}  // namespace

extern "C" int iie_attn_decode_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                                   int32_t *vcache_dev, long long pos, const int *pos_dev, long long window, const int64_t *cos_dev,
                                   const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim,
                                   long long cache_rows, int fa, long long inv_sqrt, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !q_dev || !k_dev || !v_dev || !kcache_dev || !vcache_dev || !out_dev || n_heads <= 0 || head_dim <= 0 ||
        cache_rows <= 0 || fa < 1 || fa > 29) return 1;
    AttnArgs a = {};
    a.q = q_dev; a.k = k_dev; a.v = v_dev; a.kcache = kcache_dev; a.vcache = vcache_dev; a.pos = pos;
    a.pos_dev = pos_dev; a.window = window; a.lo = 0; a.Lmax = cache_rows;
    a.cos = cos_dev; a.sin = sin_dev; a.rope = rope; a.H = n_heads; a.Hkv = n_kv; a.hd = head_dim;
    attn_consts(a, fa, inv_sqrt);
    if (!attn_scratch(a, (cudaStream_t)stream)) return 1;
    a.out = out_dev; a.flags = g_flags;
    const cudaError_t e = launch_attn_decode(a, (cudaStream_t)stream);
    if (e != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int iie_attn_prefill_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                                    int32_t *vcache_dev, long long start, long long tokens, long long window,
                                    const int64_t *cos_dev, const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim,
                                    long long cache_rows, int fa, long long inv_sqrt, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !q_dev || !k_dev || !v_dev || !kcache_dev || !vcache_dev || !out_dev || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 ||
        cache_rows <= 0 || fa < 1 || fa > 29 || start < 0 || tokens <= 0 || start + tokens > cache_rows) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    const long long Ls = (start + tokens + 63) / 64 * 64;
    // tokens in slabs so that the per-token score rows stay within a few GB
    long long slab = (4LL << 30) / ((long long)n_heads * Ls * 12);
    slab = slab < 1 ? 1 : (slab > tokens ? tokens : (slab > 65535 ? 65535 : slab));
    // own scratch roles: a captured decode graph keeps the single-token buffers' addresses
    int64_t *scores = (int64_t *)ensure(R_PSCORES, (size_t)slab * n_heads * Ls * 8);
    int32_t *e = (int32_t *)ensure(R_PEXP, (size_t)slab * n_heads * Ls * 4);
    uint8_t *st = (uint8_t *)ensure(R_PSTAT, (size_t)slab * n_heads * 16);
    if (!scores || !e || !st) return 1;
    for (long long t0 = 0; t0 < tokens; t0 += slab) {
        AttnArgs a = {};
        a.batch = (int)(tokens - t0 < slab ? tokens - t0 : slab);
        a.q = q_dev + t0 * n_heads * head_dim; a.k = k_dev + t0 * n_kv * head_dim; a.v = v_dev + t0 * n_kv * head_dim;
        a.kcache = kcache_dev; a.vcache = vcache_dev; a.pos = start + t0; a.window = window; a.Lmax = cache_rows; a.Ls = Ls;
        a.cos = cos_dev; a.sin = sin_dev; a.rope = rope; a.H = n_heads; a.Hkv = n_kv; a.hd = head_dim;
        attn_consts(a, fa, inv_sqrt);
        a.scores = scores; a.e = e; a.hmax = (long long *)st; a.Z = (unsigned long long *)(st + (size_t)slab * n_heads * 8);
        a.out = out_dev + t0 * n_heads * head_dim; a.flags = g_flags;
        if (launch_attn_prefill(a, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    }
    return 0;
}

extern "C" int iie_attn_decode_batch_dev(const int64_t *q_dev, const int64_t *k_dev, const int64_t *v_dev, int32_t *kcache_dev,
                                         int32_t *vcache_dev, long long pos, long long n_seqs, long long seq_stride, long long window,
                                         const int64_t *cos_dev, const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim,
                                         long long cache_rows, int fa, long long inv_sqrt, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !q_dev || !k_dev || !v_dev || !kcache_dev || !vcache_dev || !out_dev || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 ||
        cache_rows <= 0 || fa < 1 || fa > 29 || pos < 0 || pos >= cache_rows || n_seqs <= 0 || n_seqs > 65535 ||
        seq_stride < (long long)n_kv * cache_rows * head_dim) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    const long long Ls = (pos + 1 + 63) / 64 * 64;
    // scratch roles of their own (a captured single-token step keeps the addresses of the single-token buffers)
    int64_t *scores = (int64_t *)ensure(R_BSCORES, (size_t)n_seqs * n_heads * Ls * 8);
    int32_t *e = (int32_t *)ensure(R_BEXP, (size_t)n_seqs * n_heads * Ls * 4);
    uint8_t *st = (uint8_t *)ensure(R_BSTAT, (size_t)n_seqs * n_heads * 16);
    if (!scores || !e || !st) return 1;
    AttnArgs a = {};
    a.batch = (int)n_seqs; a.seq_stride = seq_stride;
    a.q = q_dev; a.k = k_dev; a.v = v_dev; a.kcache = kcache_dev; a.vcache = vcache_dev; a.pos = pos; a.window = window;
    a.Lmax = cache_rows; a.Ls = Ls; a.cos = cos_dev; a.sin = sin_dev; a.rope = rope; a.H = n_heads; a.Hkv = n_kv; a.hd = head_dim;
    attn_consts(a, fa, inv_sqrt);
    a.scores = scores; a.e = e; a.hmax = (long long *)st; a.Z = (unsigned long long *)(st + (size_t)n_seqs * n_heads * 8);
    a.out = out_dev; a.flags = g_flags;
    // few sequences leave most SMs idle in the probability x value pass: share each pair's chunks over up to eight CTAs
    const long long pairs = n_seqs * n_kv;
    int splits = (int)std::min<long long>(8, std::min<long long>(Ls / 64, (2368 + pairs - 1) / pairs));   // about two CTAs per SM, four waves
    if (splits > 1) {
        a.pv_part = (long long *)ensure(R_BPART, (size_t)n_seqs * splits * n_heads * head_dim * 8);
        if (!a.pv_part) return 1;
        a.pv_splits = splits;
    }
    if (launch_attn_prefill(a, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
}

// ---- attention bank (north-mini-code/tools/nmc_qk_cuda.cu:877-1551): request-scoped K/V rows on the device and the
// single-token attention sublayer on a normalised hidden row: Q/K/V products, optional interleaved RoPE, K/V append,
// exact softmax attention, O product.  K/V rows are kept as int32; a value that does not fit raises the guard
// (status 3, layer poisoned) where the reference's own guards are wider.
namespace {
// Expert bindings of one layer of a request (retained-layer executor): which registered triplets the request may use.
struct BankExperts {
    int experts = 0, used = 0;
    long long e_ffn = 0;
    int gate_q = -1, down_q = -1;                  // one block format per layer for gate/up and one for down
    unsigned maxd_gate = 0, maxdmin_gate = 0, maxd_down = 0, maxdmin_down = 0;
    std::vector<long long> gate_h, up_h, down_h;   // -1 = unbound
    const uint8_t **tabs = nullptr;                // device [3][experts]: gate, up, down pointers
    unsigned char *bound = nullptr;                // device [experts]
    std::vector<int> cold;                         // selected by the pending begin and still unbound
};
struct BankLayer {
    int32_t *k = nullptr, *v = nullptr; long long length = 0; bool poisoned = false, wide = false;
    BankExperts moe;
};
// Rows a request keeps on the device between begin and continue and from one layer to the next.
struct BankScratch {
    void *base = nullptr; size_t bytes = 0;
    int experts = 0, used = 0;                     // sized for
    int64_t *residual[2] = {nullptr, nullptr}, *hn = nullptr, *attn = nullptr, *logits = nullptr, *gates = nullptr;
    int *ids = nullptr, *cold = nullptr, *cells = nullptr;
    int8_t *hl = nullptr;
};
struct Bank {
    bool live = false;
    int n_layers = 0, heads = 0, n_kv = 0, head_dim = 0, fa = 0;
    long long max_length = 0, d_model = 0;
    int64_t *cos = nullptr, *sin = nullptr;
    std::vector<BankLayer> layers;
    BankScratch sc;
    bool pending = false, has_residual = false;
    int pending_layer = -1, retained_layer = -1, slot = 0;
};
std::vector<Bank> g_banks;

bool valid_bank(long long h) { return h >= 0 && (size_t)h < g_banks.size() && g_banks[(size_t)h].live; }

void destroy_bank(Bank &b) {
    cudaDeviceSynchronize();
    for (auto &l : b.layers) {
        if (l.k) cudaFree(l.k);
        if (l.v) cudaFree(l.v);
        if (l.moe.tabs) cudaFree(l.moe.tabs);
        if (l.moe.bound) cudaFree(l.moe.bound);
    }
    if (b.sc.base) cudaFree(b.sc.base);
    if (b.cos) cudaFree(b.cos);
    if (b.sin) cudaFree(b.sin);
    b = Bank();
}

bool ensure_bank_layer(Bank &b, BankLayer &l) {
    if (l.k && l.v) return true;
    const size_t bytes = (size_t)b.n_kv * (size_t)b.max_length * (size_t)b.head_dim * sizeof(int32_t);
    if (cudaMalloc(&l.k, bytes) != cudaSuccess || cudaMalloc(&l.v, bytes) != cudaSuccess) {
        cudaGetLastError();
        if (l.k) cudaFree(l.k);
        l.k = l.v = nullptr;
        return false;
    }
    return true;
}
}  // namespace

extern "C" long long qk_attention_bank_create(int n_layers, long long max_length, long long d_model, int heads, int n_kv,
                                              int head_dim, int fa, const int64_t *cos, const int64_t *sin) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!cos || !sin || n_layers <= 0 || max_length <= 0 || d_model <= 0 || d_model % 256 != 0 || heads <= 0 || n_kv <= 0 ||
        heads % n_kv != 0 || head_dim <= 0 || head_dim % 2 != 0 || fa < 1 || fa > 29 || ((long long)heads * head_dim) % 256 != 0 ||
        max_length > (1LL << 30) || !attn_shape_ok(heads, n_kv, head_dim) || !init()) return -1;
    Bank b;
    const size_t table = (size_t)max_length * (size_t)(head_dim / 2) * 8;
    if (cudaMalloc(&b.cos, table) != cudaSuccess || cudaMalloc(&b.sin, table) != cudaSuccess ||
        cudaMemcpy(b.cos, cos, table, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(b.sin, sin, table, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        if (b.cos) cudaFree(b.cos);
        if (b.sin) cudaFree(b.sin);
        return -1;
    }
    b.live = true; b.n_layers = n_layers; b.max_length = max_length; b.d_model = d_model; b.heads = heads; b.n_kv = n_kv;
    b.head_dim = head_dim; b.fa = fa; b.layers.resize((size_t)n_layers);
    size_t slot = g_banks.size();
    for (size_t i = 0; i < g_banks.size(); i++) if (!g_banks[i].live) { slot = i; break; }
    if (slot == g_banks.size()) g_banks.push_back(Bank());
    g_banks[slot] = std::move(b);
    return (long long)slot;
}

extern "C" int qk_attention_bank_reset(long long h) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_bank(h)) return 1;
    Bank &b = g_banks[(size_t)h];
    for (auto &l : b.layers) { l.length = 0; l.poisoned = false; l.wide = false; l.moe.cold.clear(); }
    b.pending = false; b.has_residual = false; b.pending_layer = -1; b.retained_layer = -1; b.slot = 0;
    return 0;
}

extern "C" void qk_attention_bank_destroy(long long h) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (valid_bank(h)) destroy_bank(g_banks[(size_t)h]);
}

extern "C" int qk_attention_bank_import(long long h, int layer, const int64_t *k, const int64_t *v, long long length) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_bank(h)) return 1;
    Bank &b = g_banks[(size_t)h];
    if (!k || !v || b.pending || layer < 0 || layer >= b.n_layers || length < 0 || length > b.max_length || b.layers[(size_t)layer].poisoned ||
        !ensure_bank_layer(b, b.layers[(size_t)layer])) return 1;
    BankLayer &l = b.layers[(size_t)layer];
    l.wide = false;                                          // describes the rows imported by THIS call only
    const size_t per_head = (size_t)length * (size_t)b.head_dim;
    if (per_head) {
        // narrow on the host: a value outside int32 cannot be held, so the next apply on this layer reports the guard
        std::vector<int32_t> kn((size_t)b.n_kv * per_head), vn((size_t)b.n_kv * per_head);
        for (size_t i = 0; i < kn.size(); i++) {
            if (k[i] < INT32_MIN || k[i] > INT32_MAX || v[i] < INT32_MIN || v[i] > INT32_MAX) l.wide = true;
            kn[i] = (int32_t)k[i]; vn[i] = (int32_t)v[i];
        }
        for (int head = 0; head < b.n_kv; head++) {
            const size_t src = (size_t)head * per_head, dst = (size_t)head * (size_t)b.max_length * (size_t)b.head_dim;
            if (cudaMemcpy(l.k + dst, kn.data() + src, per_head * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
                cudaMemcpy(l.v + dst, vn.data() + src, per_head * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
                cudaGetLastError(); l.poisoned = true; return 1;
            }
        }
    }
    l.length = length;
    return 0;
}

extern "C" int qk_attention_bank_apply(long long h, int layer, long long qh, long long kh, long long vh, long long oh,
                                       const int64_t *x, int fw, int window, int rope, long long inv_sqrt,
                                       long long output_capacity, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_bank(h) || !x || !out || output_capacity <= 0) return 1;
    Bank &b = g_banks[(size_t)h];
    const long long d = b.d_model, qd = (long long)b.heads * b.head_dim, kd = (long long)b.n_kv * b.head_dim;
    if (output_capacity < d || b.pending || layer < 0 || layer >= b.n_layers || !valid_q(qh) || !valid_q(kh) || !valid_q(vh) || !valid_q(oh) ||
        window == 0 || window < -1 || fw < 0 || fw > 62) return 1;
    BankLayer &l = b.layers[(size_t)layer];
    if (l.poisoned || l.length >= b.max_length || !ensure_bank_layer(b, l)) return 1;
    const Weight &wq = g_w[qh], &wk = g_w[kh], &wv = g_w[vh], &wo = g_w[oh];
    if (wq.nb != d / 256 || wk.nb != d / 256 || wv.nb != d / 256 || wq.out_f != qd || wk.out_f != kd || wv.out_f != kd ||
        wo.nb != qd / 256 || wo.out_f != d) return 1;
    if (l.wide) { l.poisoned = true; return 3; }            // imported rows did not fit the bank's int32 storage
    int64_t *xd = (int64_t *)ensure(R_X, (size_t)d * 8);
    int64_t *qkv = (int64_t *)ensure(R_TMP0, (size_t)(qd + 2 * kd) * 8);
    int64_t *att = (int64_t *)ensure(R_TMP2, (size_t)qd * 8);
    int64_t *od = (int64_t *)ensure(R_OUT, (size_t)d * 8);
    int8_t *xl = (int8_t *)ensure(R_XL, (size_t)8 * (d > qd ? d : qd));      // also holds the planes of the O product's input
    if (!xd || !qkv || !att || !od || !xl) return 1;
    // flags raised by earlier device-pointer calls belong to their caller: set aside here, put back before returning
    const int earlier = read_flags_clear();
    struct Restore { int f; ~Restore() { if (f > 0) { cudaMemcpy(g_flags, &f, sizeof(int), cudaMemcpyHostToDevice); cudaGetLastError(); } } } restore{earlier};
    if (earlier < 0 || !h2d(xd, x, (size_t)d * 8) || launch_limbs(xd, 1, d, xl, g_flags, g_stream) != cudaSuccess)
        { cudaGetLastError(); return 1; }
    bool ok = linear_dev(wq, xd, 1, fw, qkv, false, g_stream, xl) && linear_dev(wk, xd, 1, fw, qkv + qd, false, g_stream, xl) &&
              linear_dev(wv, xd, 1, fw, qkv + qd + kd, false, g_stream, xl);
    AttnArgs a = {};
    a.q = qkv; a.k = qkv + qd; a.v = qkv + qd + kd; a.kcache = l.k; a.vcache = l.v; a.pos = l.length; a.pos_dev = nullptr;
    a.window = window < 0 ? 0 : window; a.lo = 0; a.Lmax = b.max_length; a.cos = b.cos; a.sin = b.sin; a.rope = rope ? 1 : 0;
    a.H = b.heads; a.Hkv = b.n_kv; a.hd = b.head_dim;
    attn_consts(a, b.fa, inv_sqrt);
    ok = ok && attn_scratch(a, g_stream);
    a.out = att; a.flags = g_flags;
    ok = ok && launch_attn_decode(a, g_stream) == cudaSuccess;
    ok = ok && linear_dev(wo, att, 1, fw, od, false, g_stream);
    if (!ok) { cudaGetLastError(); cudaStreamSynchronize(g_stream); l.poisoned = true; return 1; }
    const int f = read_flags_clear();                       // synchronises
    if (f < 0) { l.poisoned = true; return 1; }
    if (f != 0) { l.poisoned = true; return 3; }            // a value left an exact envelope: the append is not committed
    if (!d2h(out, od, (size_t)d * 8) || !sync()) { l.poisoned = true; return 1; }
    l.length++;
    return 0;
}

extern "C" unsigned long long qk_attention_bank_workspace_bytes(long long h) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_bank(h)) return ~0ULL;
    const Bank &b = g_banks[(size_t)h];
    unsigned long long total = 2ULL * (unsigned long long)b.max_length * (unsigned long long)(b.head_dim / 2) * 8ULL;
    for (const auto &l : b.layers) {
        if (l.k) total += 2ULL * (unsigned long long)b.n_kv * (unsigned long long)b.max_length * (unsigned long long)b.head_dim * 4ULL;
        if (l.moe.experts > 0) total += (unsigned long long)l.moe.experts * (3ULL * sizeof(void *) + 1ULL);
    }
    return total + b.sc.bytes;
}

// ---- retained-layer executor over the bank (north-mini-code/tools/nmc_qk_cuda.cu:932-1028 configure / bind, 1553-1766
// begin / continue / export; bridge north-mini-code/src/nmc/qk_cuda.py:571-700).  A decode token walks consecutive MoE
// layers with the residual row, the normalised row, the routing and the attention row kept on the device:
//   begin    = norm + dense router + top-k + sigmoid gates + attention sublayer (K/V appended); returns only the
//              selected experts that have no binding yet ("cold"), so the caller can upload exactly those;
//   continue = expert stage of the selected (now bound) experts + residual + attention row -> next residual,
//              kept on the device (publish = 0) or copied out (publish = 1).
// Copies back to the host per layer: the flag word and [count | cold ids] in begin, the flag word in continue.
// Narrower than the reference, on the refusing side: one block format per layer for gate/up and one for down (a binding
// with another format returns 1); int32 K/V rows and eight-digit activations as in qk_attention_bank_apply (status 3).
namespace {
bool bank_scratch(Bank &b, int experts, int used) {
    BankScratch &sc = b.sc;
    if (sc.base && sc.experts >= experts && sc.used >= used) return true;
    experts = std::max(experts, sc.experts); used = std::max(used, sc.used);
    const size_t d = (size_t)b.d_model;
    auto up = [](size_t n) { return (n + 255) & ~(size_t)255; };
    const size_t row = up(d * 8);
    const size_t bytes = 4 * row + up((size_t)experts * 8) + up((size_t)used * 8) + up((size_t)used * 4) + up((size_t)(used + 1) * 4) + 256 + up(8 * d);
    char *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return false; }
    prof(PM_ALLOC_CALLS); prof(PM_ALLOC_BYTES, bytes);
    BankScratch n;
    n.base = p; n.bytes = bytes; n.experts = experts; n.used = used;
    n.residual[0] = (int64_t *)p; p += row; n.residual[1] = (int64_t *)p; p += row; n.hn = (int64_t *)p; p += row; n.attn = (int64_t *)p; p += row;
    n.logits = (int64_t *)p; p += up((size_t)experts * 8); n.gates = (int64_t *)p; p += up((size_t)used * 8);
    n.ids = (int *)p; p += up((size_t)used * 4); n.cold = (int *)p; p += up((size_t)(used + 1) * 4); n.cells = (int *)p; p += 256;
    n.hl = (int8_t *)p;
    if (sc.base) {                                   // a wider layer was configured later: the residual rows move along
        cudaStreamSynchronize(g_stream);
        if (cudaMemcpy(n.residual[0], sc.residual[0], d * 8, cudaMemcpyDeviceToDevice) != cudaSuccess ||
            cudaMemcpy(n.residual[1], sc.residual[1], d * 8, cudaMemcpyDeviceToDevice) != cudaSuccess) {
            cudaGetLastError(); cudaFree(n.base); return false;
        }
        cudaFree(sc.base); prof(PM_FREE_CALLS);
    }
    sc = n;
    return true;
}

// flag word -> host, counted like every other copy back to the host
int bank_read_flags() {
    prof(PM_D2H_CALLS); prof(PM_D2H_BYTES, sizeof(int));
    return read_flags_clear();
}
}  // namespace

extern "C" int qk_attention_bank_moe_configure(long long h, int layer, int experts, int used, long long d_model, long long expert_ffn) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!valid_bank(h) || layer < 0 || experts <= 0 || experts > 1024 || used <= 0 || used > experts || used > 64 || d_model <= 0 ||
        expert_ffn <= 0 || d_model % 256 != 0 || expert_ffn % 256 != 0) return 1;
    Bank &b = g_banks[(size_t)h];
    if (layer >= b.n_layers || d_model != b.d_model || b.pending || b.layers[(size_t)layer].poisoned) return 1;
    BankExperts &m = b.layers[(size_t)layer].moe;
    if (m.experts) return (m.experts == experts && m.used == used && m.e_ffn == expert_ffn) ? 0 : 1;
    const uint8_t **tabs = nullptr; unsigned char *bound = nullptr;
    if (cudaMalloc(&tabs, (size_t)3 * experts * sizeof(void *)) != cudaSuccess || cudaMalloc(&bound, (size_t)experts) != cudaSuccess ||
        cudaMemset(tabs, 0, (size_t)3 * experts * sizeof(void *)) != cudaSuccess || cudaMemset(bound, 0, (size_t)experts) != cudaSuccess) {
        cudaGetLastError();
        if (tabs) cudaFree(tabs);
        if (bound) cudaFree(bound);
        return 1;
    }
    prof(PM_ALLOC_CALLS, 2); prof(PM_ALLOC_BYTES, (size_t)experts * (3 * sizeof(void *) + 1));
    m.tabs = tabs; m.bound = bound; m.experts = experts; m.used = used; m.e_ffn = expert_ffn;
    m.gate_h.assign((size_t)experts, -1); m.up_h.assign((size_t)experts, -1); m.down_h.assign((size_t)experts, -1);
    return 0;
}

extern "C" int qk_attention_bank_moe_bind(long long h, int layer, int expert, long long gate_h, long long up_h, long long down_h) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!valid_bank(h) || layer < 0) return 1;
    Bank &b = g_banks[(size_t)h];
    if (layer >= b.n_layers || b.layers[(size_t)layer].poisoned) return 1;
    BankLayer &l = b.layers[(size_t)layer];
    BankExperts &m = l.moe;
    if (expert < 0 || expert >= m.experts || !valid_q(gate_h) || !valid_q(up_h) || !valid_q(down_h)) return 1;
    const Weight &g = g_w[gate_h], &u = g_w[up_h], &dn = g_w[down_h];
    if (g.out_f != m.e_ffn || g.nb != b.d_model / 256 || u.out_f != m.e_ffn || u.nb != b.d_model / 256 || dn.out_f != b.d_model ||
        dn.nb != m.e_ffn / 256 || g.qtype != u.qtype) return 1;
    auto retire = [&]() {
        if (b.pending && b.pending_layer == layer) m.cold.erase(std::remove(m.cold.begin(), m.cold.end(), expert), m.cold.end());
    };
    if (m.gate_h[(size_t)expert] >= 0) {
        if (m.gate_h[(size_t)expert] != gate_h || m.up_h[(size_t)expert] != up_h || m.down_h[(size_t)expert] != down_h) return 1;
        retire();
        return 0;
    }
    if ((m.gate_q >= 0 && (m.gate_q != g.qtype || m.down_q != dn.qtype))) return 1;
    const void *pg = g.d, *pu = u.d, *pd = dn.d;
    const unsigned char one = 1;
    // the bound byte goes last: a failed copy cannot leave a half-written triplet selectable
    if (cudaMemcpyAsync(m.tabs + expert, &pg, sizeof(void *), cudaMemcpyHostToDevice, g_stream) != cudaSuccess ||
        cudaMemcpyAsync(m.tabs + m.experts + expert, &pu, sizeof(void *), cudaMemcpyHostToDevice, g_stream) != cudaSuccess ||
        cudaMemcpyAsync(m.tabs + 2 * m.experts + expert, &pd, sizeof(void *), cudaMemcpyHostToDevice, g_stream) != cudaSuccess ||
        cudaMemcpyAsync(m.bound + expert, &one, 1, cudaMemcpyHostToDevice, g_stream) != cudaSuccess || !sync()) {
        cudaGetLastError(); l.poisoned = true; return 1;
    }
    m.gate_q = g.qtype; m.down_q = dn.qtype;
    m.maxd_gate = std::max({m.maxd_gate, g.maxd, u.maxd}); m.maxdmin_gate = std::max({m.maxdmin_gate, g.maxdmin, u.maxdmin});
    m.maxd_down = std::max(m.maxd_down, dn.maxd); m.maxdmin_down = std::max(m.maxdmin_down, dn.maxdmin);
    m.gate_h[(size_t)expert] = gate_h; m.up_h[(size_t)expert] = up_h; m.down_h[(size_t)expert] = down_h;
    retire();
    return 0;
}

extern "C" int qk_attention_bank_moe_begin(long long h, int layer, long long gain_h, long long router_h, long long qh, long long kh,
                                           long long vh, long long oh, const int64_t *x, int use_retained, int fw,
                                           unsigned long long eps, int window, int rope, long long inv_sqrt, int cold_capacity,
                                           int *cold_count_out, int *cold_ids_out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!valid_bank(h) || layer < 0 || !cold_count_out || !cold_ids_out || use_retained < 0 || use_retained > 1 || fw < 0 || fw > 62 ||
        window == 0 || window < -1) return 1;
    Bank &b = g_banks[(size_t)h];
    if (layer >= b.n_layers || b.pending || !valid_i64(gain_h) || !valid_i64(router_h)) return 1;
    BankLayer &l = b.layers[(size_t)layer];
    BankExperts &m = l.moe;
    const Weight &gain = g_w[gain_h], &router = g_w[router_h];
    const long long d = b.d_model, qd = (long long)b.heads * b.head_dim, kd = (long long)b.n_kv * b.head_dim;
    if (l.poisoned || m.experts <= 0 || !m.cold.empty() || cold_capacity < m.used || gain.out_f != 1 || gain.nb != d ||
        router.out_f != m.experts || router.nb != d) return 1;
    if ((!use_retained && !x) || (use_retained && (!b.has_residual || b.retained_layer + 1 != layer))) return 1;
    // the projections are checked before anything is queued: a refused begin leaves the request as it was
    if (!valid_q(qh) || !valid_q(kh) || !valid_q(vh) || !valid_q(oh) || l.length >= b.max_length) return 1;
    const Weight &wq = g_w[qh], &wk = g_w[kh], &wv = g_w[vh], &wo = g_w[oh];
    if (wq.nb != d / 256 || wk.nb != d / 256 || wv.nb != d / 256 || wq.out_f != qd || wk.out_f != kd || wv.out_f != kd ||
        wo.nb != qd / 256 || wo.out_f != d) return 1;
    if (!ensure_bank_layer(b, l) || !bank_scratch(b, m.experts, m.used)) return 1;
    if (l.wide) { l.poisoned = true; return 3; }
    BankScratch &sc = b.sc;
    int64_t *qkv = (int64_t *)ensure(R_TMP0, (size_t)(qd + 2 * kd) * 8);
    int64_t *att = (int64_t *)ensure(R_TMP2, (size_t)qd * 8);
    if (!qkv || !att) return 1;
    const int earlier = read_flags_clear();
    struct Restore { int f; ~Restore() { if (f > 0) { cudaMemcpy(g_flags, &f, sizeof(int), cudaMemcpyHostToDevice); cudaGetLastError(); } } } restore{earlier};
    if (earlier < 0) return 1;
    int64_t *residual = sc.residual[use_retained ? b.slot : 0];
    if (!use_retained) {
        if (!h2d(residual, x, (size_t)d * 8)) { cudaGetLastError(); return 1; }
        b.slot = 0;
    }
    bool ok = cudaMemsetAsync(sc.cells, 0, 4 * sizeof(int), g_stream) == cudaSuccess &&
              launch_rmsnorm(residual, 1, d, (const int64_t *)gain.d, b.fa, eps, sc.hn, g_flags, g_stream) == cudaSuccess &&
              launch_limbs(sc.hn, 1, d, sc.hl, g_flags, g_stream, sc.cells) == cudaSuccess &&
              launch_exact_dense((const int64_t *)router.d, m.experts, d, sc.hn, 1, fw, sc.logits, g_flags, g_stream) == cudaSuccess &&
              launch_topk(sc.logits, 1, m.experts, m.used, b.fa, sc.ids, sc.gates, g_stream) == cudaSuccess &&
              launch_cold_routes(sc.ids, m.used, m.bound, m.experts, sc.cold, g_flags, g_stream) == cudaSuccess;
    ok = ok && linear_dev(wq, sc.hn, 1, fw, qkv, false, g_stream, sc.hl) && linear_dev(wk, sc.hn, 1, fw, qkv + qd, false, g_stream, sc.hl) &&
         linear_dev(wv, sc.hn, 1, fw, qkv + qd + kd, false, g_stream, sc.hl);
    AttnArgs a = {};
    a.q = qkv; a.k = qkv + qd; a.v = qkv + qd + kd; a.kcache = l.k; a.vcache = l.v; a.pos = l.length; a.pos_dev = nullptr;
    a.window = window < 0 ? 0 : window; a.lo = 0; a.Lmax = b.max_length; a.cos = b.cos; a.sin = b.sin; a.rope = rope ? 1 : 0;
    a.H = b.heads; a.Hkv = b.n_kv; a.hd = b.head_dim;
    attn_consts(a, b.fa, inv_sqrt);
    ok = ok && attn_scratch(a, g_stream);
    a.out = att; a.flags = g_flags;
    ok = ok && launch_attn_decode(a, g_stream) == cudaSuccess;
    ok = ok && linear_dev(wo, att, 1, fw, sc.attn, false, g_stream);
    if (!ok) { cudaGetLastError(); cudaStreamSynchronize(g_stream); l.poisoned = true; return 1; }
    const int f = bank_read_flags();                       // synchronises: routing, attention and the append are judged together
    if (f < 0) { l.poisoned = true; return 1; }
    if (f != 0) { l.poisoned = true; return 3; }
    std::vector<int> cold((size_t)m.used + 1, 0);
    if (!d2h(cold.data(), sc.cold, cold.size() * sizeof(int)) || !sync() || cold[0] < 0 || cold[0] > m.used) {
        cudaGetLastError(); l.poisoned = true; return 1;
    }
    m.cold.assign(cold.begin() + 1, cold.begin() + 1 + cold[0]);
    for (int i = 0; i < cold[0]; i++) cold_ids_out[i] = cold[(size_t)i + 1];
    *cold_count_out = cold[0];
    l.length++;
    b.has_residual = true; b.pending = true; b.pending_layer = layer;
    return 0;
}

extern "C" int qk_attention_bank_moe_continue(long long h, int layer, int fw, int publish, long long output_capacity, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS); prof(PM_MOE);
    if (!valid_bank(h) || layer < 0 || fw < 0 || fw > 62 || publish < 0 || publish > 1 || (publish && (!out || output_capacity <= 0))) return 1;
    Bank &b = g_banks[(size_t)h];
    if (layer >= b.n_layers || !b.pending || b.pending_layer != layer) return 1;
    BankLayer &l = b.layers[(size_t)layer];
    BankExperts &m = l.moe;
    const long long d = b.d_model;
    if (l.poisoned || m.experts <= 0 || !b.sc.base || (publish && output_capacity < d)) return 1;
    if (!m.cold.empty()) return 4;                            // begin's cold set has not been bound completely
    BankScratch &sc = b.sc;
    const int k = m.used, E = m.experts;
    int64_t *residual = sc.residual[b.slot], *next = sc.residual[b.slot ^ 1];
    const int earlier = read_flags_clear();
    struct Restore { int f; ~Restore() { if (f > 0) { cudaMemcpy(g_flags, &f, sizeof(int), cudaMemcpyHostToDevice); cudaGetLastError(); } } } restore{earlier};
    if (earlier < 0) return 1;
    bool ok = launch_add_rows(residual, sc.attn, next, d, g_stream) == cudaSuccess;
    if (fast_envelope(m.gate_q, d / 256, m.maxd_gate, m.maxdmin_gate, fw) && fast_envelope(m.down_q, m.e_ffn / 256, m.maxd_down, m.maxdmin_down, fw)) {
        int8_t *gul = (int8_t *)ensure(R_GUL, (size_t)k * 8 * m.e_ffn);
        ok = ok && gul;
        StreamArgs ga = {};
        ga.wa = m.tabs; ga.wb = m.tabs + E; ga.sel = sc.ids; ga.n_sel = k; ga.out_f = m.e_ffn; ga.n_blocks = d / 256; ga.fw = fw; ga.fa = b.fa;
        ga.xl = sc.hl; ga.x_per_sel = 0; ga.x_nl = sc.cells; ga.out = nullptr; ga.out_limbs = gul; ga.out_nl = sc.cells + 1; ga.flags = g_flags;
        ga.fast = small_scales(m.maxd_gate, m.maxdmin_gate, fw);
        StreamArgs da = {};
        da.wa = m.tabs + 2 * E; da.wb = da.wa; da.sel = sc.ids; da.n_sel = k; da.out_f = d; da.n_blocks = m.e_ffn / 256; da.fw = fw; da.fa = b.fa;
        da.xl = gul; da.x_per_sel = 1; da.x_nl = sc.cells + 1; da.out = next; da.gates = sc.gates; da.flags = g_flags;
        da.fast = small_scales(m.maxd_down, m.maxdmin_down, fw);
        ok = ok && launch_stream(m.gate_q, MODE_GATEUP, ga, g_stream) == cudaSuccess && launch_stream(m.down_q, MODE_DOWN, da, g_stream) == cudaSuccess;
    } else {
        // block scales beyond the streamed kernels' envelope: the per-weight 128-bit products, selected on the host
        std::vector<int> ids((size_t)k);
        ok = ok && d2h(ids.data(), sc.ids, (size_t)k * sizeof(int)) && sync();
        std::vector<const Weight *> gw, uw, dw;
        for (int i = 0; ok && i < k; i++) {
            const int e = ids[(size_t)i];
            if (e < 0 || e >= E || m.gate_h[(size_t)e] < 0) { ok = false; break; }
            gw.push_back(&g_w[m.gate_h[(size_t)e]]); uw.push_back(&g_w[m.up_h[(size_t)e]]); dw.push_back(&g_w[m.down_h[(size_t)e]]);
        }
        int64_t *moe = ok ? (int64_t *)ensure(R_OUT, (size_t)d * 8) : nullptr;
        ok = ok && moe && moe_exact_pairs(gw, uw, dw, sc.hn, std::vector<int>((size_t)k, 0), sc.gates, 1, k, d, m.e_ffn, b.fa, fw, moe) &&
             launch_add_rows(next, moe, next, d, g_stream) == cudaSuccess;
    }
    if (!ok) { cudaGetLastError(); cudaStreamSynchronize(g_stream); l.poisoned = true; return 1; }
    const int f = bank_read_flags();
    if (f < 0) { l.poisoned = true; return 1; }
    if (f != 0) { l.poisoned = true; return 3; }
    if (publish && (!d2h(out, next, (size_t)d * 8) || !sync())) { cudaGetLastError(); l.poisoned = true; return 1; }
    b.slot ^= 1; b.has_residual = true; b.retained_layer = layer; b.pending = false; b.pending_layer = -1;
    return 0;
}

extern "C" int qk_attention_bank_moe_export(long long h, long long output_capacity, int64_t *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!valid_bank(h) || !out || output_capacity <= 0) return 1;
    Bank &b = g_banks[(size_t)h];
    if (b.pending || !b.has_residual || b.retained_layer < 0 || !b.sc.base || output_capacity < b.d_model) return 1;
    if (!d2h(out, b.sc.residual[b.slot], (size_t)b.d_model * 8) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int iie_attn_block_dev(long long wqkv_h, long long wo_h, int64_t *x_dev, int32_t *kcache_dev, int32_t *vcache_dev,
                                  long long pos, const int *pos_dev, long long window, const int64_t *cos_dev,
                                  const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim, long long cache_rows,
                                  int fa, int fw, long long inv_sqrt, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !valid_q(wqkv_h) || !valid_q(wo_h) || !x_dev || !kcache_dev || !vcache_dev || n_heads <= 0 || n_kv <= 0 ||
        head_dim <= 0 || cache_rows <= 0 || fa < 1 || fa > 29) return 1;
    const Weight &wqkv = g_w[wqkv_h], &wo = g_w[wo_h];
    const long long d = wqkv.nb * 256, qd = (long long)n_heads * head_dim, kd = (long long)n_kv * head_dim;
    if (wqkv.out_f != qd + 2 * kd || wo.nb * 256 != qd || wo.out_f != d || g_hl_d != d) return 1;   // g_hl_d: the digit planes on hand
    if (!fast_envelope(wqkv.qtype, wqkv.nb, wqkv.maxd, wqkv.maxdmin, fw) || !fast_envelope(wo.qtype, wo.nb, wo.maxd, wo.maxdmin, fw)) return 3;
    cudaStream_t s = (cudaStream_t)stream;
    const int8_t *hl = (const int8_t *)g_buf[R_XL].p;
    int64_t *qkv = (int64_t *)ensure(R_TMP0, (size_t)(qd + 2 * kd) * 8);
    int8_t *al = (int8_t *)ensure(R_TMP1, (size_t)8 * qd);
    if (!hl || !qkv || !al) return 1;
    StreamArgs sa = {};
    sa.wa = wqkv.cell; sa.wb = wqkv.cell; sa.n_sel = 1; sa.out_f = wqkv.out_f; sa.n_blocks = wqkv.nb; sa.fw = fw; sa.fa = fa;
    sa.xl = hl; sa.x_per_sel = 0; sa.x_nl = g_cells; sa.out = qkv; sa.flags = g_flags;
    sa.fast = small_scales(wqkv.maxd, wqkv.maxdmin, fw); sa.pdl = g_pdl; sa.early_weights = sa.pdl;   // fixed weight pointer: request before the wait
    if (launch_stream(wqkv.qtype, MODE_LINEAR, sa, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    AttnArgs a = {};
    a.q = qkv; a.k = qkv + qd; a.v = qkv + qd + kd; a.kcache = kcache_dev; a.vcache = vcache_dev; a.pos = pos;
    a.pos_dev = pos_dev; a.window = window; a.lo = 0; a.Lmax = cache_rows;
    a.cos = cos_dev; a.sin = sin_dev; a.rope = rope; a.H = n_heads; a.Hkv = n_kv; a.hd = head_dim;
    attn_consts(a, fa, inv_sqrt);
    if (!attn_scratch(a, s)) return 1;
    int *nl_cell = g_cells + 16 + 128 * g_attn_parity;        // one count per KV head; alternate between calls
    g_attn_parity ^= 1;
    a.out = nullptr; a.out_limbs = al; a.out_nl = nl_cell; a.flags = g_flags; a.pdl = g_pdl;
    if (launch_attn_decode(a, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    // O product accumulated into the residual row: the "down" form of the streaming kernel with a unit gate
    StreamArgs oa = {};
    oa.wa = wo.cell; oa.wb = wo.cell; oa.n_sel = 1; oa.out_f = wo.out_f; oa.n_blocks = wo.nb; oa.fw = fw; oa.fa = fa;
    oa.xl = al; oa.x_per_sel = 1; oa.x_nl = nl_cell; oa.x_nl_n = n_kv <= 120 ? n_kv : 1; oa.out = x_dev; oa.gates = g_pow2 + fa; oa.flags = g_flags;
    oa.fast = small_scales(wo.maxd, wo.maxdmin, fw); oa.pdl = g_pdl; oa.early_weights = g_pdl;
    if (launch_stream(wo.qtype, MODE_DOWN, oa, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
}

// One whole parallel decoder block for one token, x += attention(h) Wo^T + moe(h) with h = rmsnorm(x, gain), as five
// launches chained by programmatic dependent launch:
//   front     every CTA normalises x and takes its share of the rows of [Wq|Wk|Wv] and of the router (one kernel
//             instead of the routing kernel followed by the fused QKV product);
//   attention cooperative single-token attention (K/V append, scores, softmax, p.V);
//   O         product accumulated into x; one more CTA of the same launch ranks the router logits (top-k, lowest index
//             among equals, sigmoid gates) on an SM the product leaves idle and leaves indices, gates and the selected
//             matrices' pointers for the two kernels behind it;
//   gate/up   expert gate and up products of the selected experts, SiLU, digit planes of the result;
//   down      weights requested before its dependency wait (the selection is final a launch earlier), gate-weighted rows
//             accumulated into x.
// Same bytes as iie_moe_block_dev followed by iie_attn_block_dev.  Status 5: this shape has no fused form (dense router,
// router and Wqkv of different block formats, more than 64 selected experts) and the two entries must be used.
extern "C" int iie_block_dev(long long layer, long long gain_h, long long wqkv_h, long long wo_h, int64_t *x_dev, int32_t *kcache_dev,
                             int32_t *vcache_dev, long long pos, const int *pos_dev, long long window, const int64_t *cos_dev,
                             const int64_t *sin_dev, int rope, int n_heads, int n_kv, int head_dim, long long cache_rows, int fa, int fw,
                             unsigned long long eps, long long inv_sqrt, int *ids_dev, int64_t *gates_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live || !valid_q(wqkv_h) || !valid_q(wo_h) || !x_dev ||
        !kcache_dev || !vcache_dev || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || cache_rows <= 0 || fa < 1 || fa > 29 ||
        fw < 0 || fw > 62) return 1;
    const MoeLayer &L = g_layers[layer];
    if (L.router < 0) return 1;
    const Weight &r = g_w[L.router], &wqkv = g_w[wqkv_h], &wo = g_w[wo_h];
    const long long d = L.d_model, qd = (long long)n_heads * head_dim, kd = (long long)n_kv * head_dim;
    const int E = L.n_experts, k = L.top_k;
    if (wqkv.nb * 256 != d || wqkv.out_f != qd + 2 * kd || wo.nb * 256 != qd || wo.out_f != d) return 1;
    if (r.qtype == QT_I64 || r.qtype != wqkv.qtype || k > 64 || E > 1024 || d > 4096 || g_stage_mask != 0) return 5;
    const int64_t *gain = nullptr;
    if (gain_h >= 0) {
        if (!valid_i64(gain_h) || g_w[gain_h].out_f != 1 || g_w[gain_h].nb != d) return 1;
        gain = (const int64_t *)g_w[gain_h].d;
    }
    if (!fast_envelope(L.gate_q, d / 256, L.maxd_gate, L.maxdmin_gate, fw) || !fast_envelope(L.down_q, L.e_ffn / 256, L.maxd_down, L.maxdmin_down, fw) ||
        !fast_envelope(wqkv.qtype, wqkv.nb, wqkv.maxd, wqkv.maxdmin, fw) || !fast_envelope(wo.qtype, wo.nb, wo.maxd, wo.maxdmin, fw) ||
        !fast_envelope(r.qtype, r.nb, r.maxd, r.maxdmin, fw)) return 3;
    cudaStream_t s = (cudaStream_t)stream;
    int8_t *hl = (int8_t *)ensure(R_XL, (size_t)8 * d);
    int64_t *lg = (int64_t *)ensure(R_LOGITS, (size_t)E * 8);
    int8_t *gul = (int8_t *)ensure(R_GUL, (size_t)k * 8 * L.e_ffn);
    int64_t *qkv = (int64_t *)ensure(R_TMP0, (size_t)(qd + 2 * kd) * 8);
    int8_t *al = (int8_t *)ensure(R_TMP1, (size_t)8 * qd);
    if (!hl || !lg || !gul || !qkv || !al) return 1;
    g_hl_d = d;
    StreamArgs f = {};
    f.wa = wqkv.cell; f.wb = r.cell; f.n_sel = 1; f.out_f = wqkv.out_f; f.out_f_b = E; f.n_blocks = d / 256; f.fw = fw; f.fa = fa;
    f.x = x_dev; f.gain = gain; f.eps = eps; f.out = qkv; f.out_b = lg; f.hl_out = hl; f.h_nl_out = g_cells; f.gu_nl_zero = g_cells + 1;
    f.pf_base = kcache_dev; f.pf_rows = cache_rows; f.pf_pos = pos; f.pf_window = window; f.pf_heads = n_kv;
    f.pf_row_bytes = head_dim * 4; f.pf_pos_dev = pos_dev;      // the key rows attention asks for first: into L2 meanwhile
    f.flags = g_flags; f.pdl = g_pdl; f.early_weights = g_pdl;
    f.fast = small_scales(std::max(wqkv.maxd, r.maxd), std::max(wqkv.maxdmin, r.maxdmin), fw);
    if (launch_stream(wqkv.qtype, MODE_FRONT, f, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    AttnArgs a = {};
    a.q = qkv; a.k = qkv + qd; a.v = qkv + qd + kd; a.kcache = kcache_dev; a.vcache = vcache_dev; a.pos = pos;
    a.pos_dev = pos_dev; a.window = window; a.lo = 0; a.Lmax = cache_rows;
    a.cos = cos_dev; a.sin = sin_dev; a.rope = rope; a.H = n_heads; a.Hkv = n_kv; a.hd = head_dim;
    attn_consts(a, fa, inv_sqrt);
    if (!attn_scratch(a, s)) return 1;
    int *nl_cell = g_cells + 16 + 128 * g_attn_parity;
    g_attn_parity ^= 1;
    a.out = nullptr; a.out_limbs = al; a.out_nl = nl_cell; a.flags = g_flags; a.pdl = g_pdl;
    if (launch_attn_decode(a, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    StreamArgs oa = {};
    oa.wa = wo.cell; oa.wb = wo.cell; oa.n_sel = 1; oa.out_f = wo.out_f; oa.n_blocks = wo.nb; oa.fw = fw; oa.fa = fa;
    oa.xl = al; oa.x_per_sel = 1; oa.x_nl = nl_cell; oa.x_nl_n = n_kv <= 120 ? n_kv : 1; oa.out = x_dev; oa.gates = g_pow2 + fa; oa.flags = g_flags;
    oa.fast = small_scales(wo.maxd, wo.maxdmin, fw); oa.pdl = g_pdl; oa.early_weights = g_pdl;
    // the ranking of the router logits (final since the front kernel) rides on an SM the O product leaves idle
    int *ids = ids_dev ? ids_dev : (int *)ensure(R_IDS, (size_t)k * sizeof(int));
    int64_t *gates = gates_dev ? gates_dev : (int64_t *)ensure(R_GATES, (size_t)k * 8);
    if (!ids || !gates) return 1;
    oa.rank_logits = lg; oa.rank_n = E; oa.rank_k = k; oa.rank_ids = ids; oa.rank_gates = gates;
    oa.rank_tabs = L.tabs; oa.rank_ptrs = g_selptr;          // k <= 64 here: the table holds 3 x 64 pointers
    if (launch_stream(wo.qtype, MODE_DOWN, oa, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    StreamArgs ga = {};
    ga.wa = L.tabs; ga.wb = L.tabs + E; ga.n_sel = k; ga.out_f = L.e_ffn; ga.n_blocks = d / 256; ga.fw = fw; ga.fa = fa;
    ga.sel = ids; ga.sel_wa = g_selptr; ga.sel_wb = g_selptr + k;
    ga.xl = hl; ga.x_per_sel = 0; ga.x_nl = g_cells; ga.out = nullptr; ga.out_limbs = gul; ga.out_nl = g_cells + 1; ga.flags = g_flags;
    ga.fast = small_scales(L.maxd_gate, L.maxdmin_gate, fw); ga.pdl = g_pdl; ga.early_weights = 0;       // the selection comes from the kernel in front
    if (launch_stream(L.gate_q, MODE_GATEUP, ga, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    StreamArgs da = {};
    da.wa = L.tabs + 2 * E; da.wb = da.wa; da.n_sel = k; da.out_f = d; da.n_blocks = L.e_ffn / 256; da.fw = fw; da.fa = fa;
    da.sel = ids; da.gates = gates; da.sel_wa = g_selptr + 2 * k;
    da.xl = gul; da.x_per_sel = 1; da.x_nl = g_cells + 1; da.out = x_dev; da.flags = g_flags;
    da.fast = small_scales(L.maxd_down, L.maxdmin_down, fw); da.pdl = g_pdl; da.early_weights = g_pdl;
    if (launch_stream(L.down_q, MODE_DOWN, da, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
}

extern "C" int iie_embed_dev(long long h, const int *token_dev, long long token, int frac, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !valid_q(h) || !out_dev || frac < 0 || frac > 40) return 1;
    const Weight &w = g_w[h];
    if (!token_dev && (token < 0 || token >= w.out_f)) return 1;
    return launch_embed_row((const uint8_t *)w.d, w.qtype, w.nb, token_dev, token, frac, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 1;
}

extern "C" int iie_argmax_dev(const int64_t *x_dev, long long n, int *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !x_dev || !out_dev || n <= 0) return 1;
    return launch_argmax(x_dev, n, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 1;
}

extern "C" int iie_embed_rows_dev(long long h, const int *tokens_dev, int rows, int frac, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !valid_q(h) || !tokens_dev || !out_dev || rows <= 0 || frac < 0 || frac > 40) return 1;
    const Weight &w = g_w[h];
    return launch_embed_rows((const uint8_t *)w.d, w.qtype, w.nb, tokens_dev, rows, frac, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 1;
}

extern "C" int iie_argmax_rows_dev(const int64_t *x_dev, long long rows, long long n, int *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !x_dev || !out_dev || n <= 0 || rows <= 0) return 1;
    return launch_argmax_rows(x_dev, rows, n, out_dev, (cudaStream_t)stream) == cudaSuccess ? 0 : 1;
}

extern "C" int iie_apply_dev(long long h, const int64_t *x_dev, long long T, int fw, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !valid_q(h) || !x_dev || !out_dev || T <= 0) return 1;
    cudaStream_t s = (cudaStream_t)stream;              // NULL is the CUDA default stream
    return linear_dev(g_w[h], x_dev, T, fw, out_dev, false, s) ? 0 : 1;
}

extern "C" int iie_flags_read_clear(void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init()) return -1;
    if (stream && cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return -1;
    return read_flags_clear();
}

extern "C" int iie_rmsnorm_dev(long long gain_h, const int64_t *x_dev, long long rows, long long width, int fa,
                               unsigned long long eps, int64_t *out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || !x_dev || !out_dev || rows <= 0 || width <= 0 || fa < 1 || fa > 29) return 1;
    const int64_t *gain = nullptr;
    if (gain_h >= 0) {
        if (!valid_i64(gain_h) || g_w[gain_h].out_f != 1 || g_w[gain_h].nb != width) return 1;
        gain = (const int64_t *)g_w[gain_h].d;
    }
    cudaStream_t s = (cudaStream_t)stream;              // NULL is the CUDA default stream
    return launch_rmsnorm(x_dev, rows, width, gain, fa, eps, out_dev, g_flags, s) == cudaSuccess ? 0 : 1;
}

extern "C" void iie_set_tc_min_tokens(long long tokens) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    g_tc_min_tokens = tokens < 2 ? 2 : tokens;
}

extern "C" void iie_set_attn_fused(int enabled) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    iie::g_attn_fused = enabled < 0 ? 0 : enabled > 2 ? 2 : enabled;
}

extern "C" void iie_set_attn_tile_tc(int enabled) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    iie::g_attn_tile_tc = enabled > 0 ? 1 : enabled < 0 ? -1 : 0;
}

extern "C" void iie_set_pdl(int enabled) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    g_pdl = enabled ? 1 : 0;
}

extern "C" void iie_profile_stage_mask(int mask) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    g_stage_mask = mask;
}

extern "C" unsigned long long iie_workspace_generation(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    return g_ws_generation;
}

extern "C" int iie_prefill_launch_counts(unsigned long long *out, int capacity) {
    if (!out || capacity < iie::PF_SHAPES) return -1;
    for (int i = 0; i < iie::PF_SHAPES; i++) out[i] = __atomic_load_n(&iie::g_prefill_launches[i], __ATOMIC_RELAXED);
    return iie::PF_SHAPES;
}

extern "C" unsigned long long iie_launch_count(void) { return __atomic_load_n(&iie::g_launches, __ATOMIC_RELAXED); }

extern "C" int iie_moe_block_dev(long long layer, long long gain_h, const int64_t *x_dev, long long T, int fa, int fw,
                                 unsigned long long eps, int64_t *out_dev, int *ids_dev, int64_t *gates_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live || !x_dev || !out_dev ||
        T <= 0 || fa < 1 || fa > 29 || g_layers[layer].router < 0) return 1;
    const MoeLayer &L = g_layers[layer];
    cudaStream_t s = (cudaStream_t)stream;              // NULL is the CUDA default stream
    if (!fast_envelope(L.gate_q, L.d_model / 256, L.maxd_gate, L.maxdmin_gate, fw) ||
        !fast_envelope(L.down_q, L.e_ffn / 256, L.maxd_down, L.maxdmin_down, fw)) return 3;
    const int64_t *gain = nullptr;
    if (gain_h >= 0) {
        if (!valid_i64(gain_h) || g_w[gain_h].out_f != 1 || g_w[gain_h].nb != L.d_model) return 1;
        gain = (const int64_t *)g_w[gain_h].d;
    }
    const size_t n = (size_t)T * L.d_model, P = (size_t)T * L.top_k;
    if (T == 1 && g_w[L.router].qtype != QT_I64 && L.d_model <= 4096 && L.top_k <= 32) {
        int *ids = ids_dev ? ids_dev : (int *)ensure(R_IDS, P * sizeof(int));
        int64_t *gates = gates_dev ? gates_dev : (int64_t *)ensure(R_GATES, P * 8);
        if (!ids || !gates) return 1;
        const int init_mode = gain ? (out_dev == x_dev ? 0 : 2) : 1;
        if (!moe_decode_token(L, x_dev, gain, fa, fw, eps, init_mode, out_dev, ids, gates, s)) { cudaGetLastError(); return 1; }
        return 0;
    }
    const int64_t *h = x_dev;
    if (gain) {
        int64_t *hd = (int64_t *)ensure(R_HNORM, n * 8);
        if (!hd || launch_rmsnorm(x_dev, T, L.d_model, gain, fa, eps, hd, g_flags, s) != cudaSuccess) return 1;
        h = hd;
        if (out_dev != x_dev && cudaMemcpyAsync(out_dev, x_dev, n * 8, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return 1;
    }
    return iie_moe_forward_dev(layer, h, T, fa, fw, gain ? 1 : 0, out_dev, ids_dev, gates_dev, s);
}

extern "C" int iie_moe_block_host(long long layer, long long gain_h, const int64_t *x, long long T, int fa, int fw,
                                  unsigned long long eps, int64_t *out, int *ids_out, int64_t *gates_out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    prof(PM_NATIVE_CALLS);
    if (!init() || layer < 0 || (size_t)layer >= g_layers.size() || !g_layers[layer].live || !x || !out || T <= 0) return 1;
    const MoeLayer &L = g_layers[layer];
    const size_t n = (size_t)T * L.d_model;
    const size_t P = (size_t)T * L.top_k;
    int64_t *xd = (int64_t *)ensure(R_X, n * 8), *od = (int64_t *)ensure(R_OUT, n * 8);
    int64_t *gd = (int64_t *)ensure(R_GATES, P * 8);
    int *idd = (int *)ensure(R_IDS, P * sizeof(int));
    if (!xd || !od || !gd || !idd || !h2d(xd, x, n * 8)) { cudaGetLastError(); return 1; }
    const int rc = iie_moe_block_dev(layer, gain_h, xd, T, fa, fw, eps, od, idd, gd, g_stream);
    if (rc != 0) { cudaGetLastError(); return rc; }
    const int f = read_flags_clear();
    if (f < 0) return 1;
    if (f) return 3;
    if (!d2h(out, od, n * 8) || (ids_out && !d2h(ids_out, idd, P * sizeof(int))) ||
        (gates_out && !d2h(gates_out, gd, P * 8)) || !sync()) { cudaGetLastError(); return 1; }
    return 0;
}

// ====================================================================================================
// Whole decode step in one launch (decode.cu)
// ====================================================================================================
namespace {
struct DecoderObj {
    bool live = false, dirty = true;
    int n_layers = 0, n_set = 0, n_ctas = 0;
    DecodeArgs a = {};                               // model-wide arguments; per-call fields are filled in by the step
    std::vector<DecodeLayer> layers;
    std::vector<bool> set;
    DecodeLayer *layers_dev = nullptr;
    uint8_t *scratch = nullptr;
    int down_q = -1;
};
std::vector<DecoderObj> g_decoders;
bool valid_decoder(long long h) { return h >= 0 && (size_t)h < g_decoders.size() && g_decoders[(size_t)h].live; }

void free_decoder(DecoderObj &d) {
    if (g_stream) cudaDeviceSynchronize();
    if (d.layers_dev) cudaFree(d.layers_dev);
    if (d.scratch) cudaFree(d.scratch);
    d = DecoderObj();
}
}  // namespace

extern "C" long long iie_decoder_create(int n_layers, int n_heads, int n_kv, int head_dim, long long window, long long cache_rows,
                                        int fa, int fw, unsigned long long eps, long long inv_sqrt, const int64_t *cos_dev,
                                        const int64_t *sin_dev) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!init() || n_layers <= 0 || n_layers > 4096 || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || cache_rows <= 0 || fa < 1 ||
        fa > 29 || fw < 24 || fw > 36 || !cos_dev || !sin_dev || window < 0) return -1;
    DecoderObj d;
    d.live = true; d.n_layers = n_layers; d.layers.resize((size_t)n_layers); d.set.assign((size_t)n_layers, false);
    d.a.n_layers = n_layers; d.a.H = n_heads; d.a.Hkv = n_kv; d.a.hd = head_dim; d.a.window = window; d.a.Lmax = cache_rows;
    d.a.fa = fa; d.a.fw = fw; d.a.eps = eps; d.a.cos = cos_dev; d.a.sin = sin_dev; d.a.flags = g_flags;
    AttnArgs tmp = {};
    attn_consts(tmp, fa, inv_sqrt);
    d.a.inv_sqrt = tmp.inv_sqrt; d.a.log2e = tmp.log2e; d.a.clip = tmp.clip;
    d.a.sig_log2e = sigmoid_log2e(fa); d.a.sig_clip = sigmoid_clip(fa);
    size_t slot = g_decoders.size();
    for (size_t i = 0; i < g_decoders.size(); i++) if (!g_decoders[i].live) { slot = i; break; }
    if (slot == g_decoders.size()) g_decoders.push_back(DecoderObj());
    g_decoders[slot] = std::move(d);
    return (long long)slot;
}

extern "C" int iie_decoder_set_layer(long long dec, int li, long long gain_h, long long moe_layer, long long wqkv_h, long long wo_h,
                                     int32_t *kcache_dev, int32_t *vcache_dev, int full) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_decoder(dec)) return 1;
    DecoderObj &d = g_decoders[(size_t)dec];
    if (li < 0 || li >= d.n_layers || moe_layer < 0 || (size_t)moe_layer >= g_layers.size() || !g_layers[moe_layer].live ||
        !valid_i64(gain_h) || !valid_q(wqkv_h) || !valid_q(wo_h) || !kcache_dev || !vcache_dev) return 1;
    const MoeLayer &L = g_layers[moe_layer];
    if (L.router < 0) return 1;
    const Weight &r = g_w[L.router], &wq = g_w[wqkv_h], &wo = g_w[wo_h], &gain = g_w[gain_h];
    const DecodeArgs &a = d.a;
    const long long qd = (long long)a.H * a.hd, kd = (long long)a.Hkv * a.hd;
    if (gain.out_f != 1 || gain.nb != L.d_model || wq.nb * 256 != L.d_model || wq.out_f != qd + 2 * kd || wo.nb * 256 != qd ||
        wo.out_f != L.d_model) return 1;
    // what the one-launch kernel carries: Q4_K router / attention / gate / up matrices with small block scales
    if (r.qtype != QT_Q4K || wq.qtype != QT_Q4K || wo.qtype != QT_Q4K || L.gate_q != QT_Q4K) return 5;
    if (!small_scales(r.maxd, r.maxdmin, a.fw) || !small_scales(wq.maxd, wq.maxdmin, a.fw) || !small_scales(wo.maxd, wo.maxdmin, a.fw) ||
        !small_scales(L.maxd_gate, L.maxdmin_gate, a.fw) || !small_scales(L.maxd_down, L.maxdmin_down, a.fw)) return 5;
    if (!fast_envelope(QT_Q4K, r.nb, r.maxd, r.maxdmin, a.fw) || !fast_envelope(QT_Q4K, wq.nb, wq.maxd, wq.maxdmin, a.fw) ||
        !fast_envelope(QT_Q4K, wo.nb, wo.maxd, wo.maxdmin, a.fw) ||
        !fast_envelope(QT_Q4K, L.d_model / 256, L.maxd_gate, L.maxdmin_gate, a.fw) ||
        !fast_envelope(L.down_q, L.e_ffn / 256, L.maxd_down, L.maxdmin_down, a.fw)) return 5;
    if (d.n_set == 0) {
        d.a.d = (int)L.d_model; d.a.E = L.n_experts; d.a.k = L.top_k; d.a.eff = (int)L.e_ffn; d.down_q = L.down_q;
        if (!decode_shape_ok(d.a.d, a.H, a.Hkv, a.hd, d.a.E, d.a.k, d.a.eff, L.down_q)) return 5;
    } else if (d.a.d != L.d_model || d.a.E != L.n_experts || d.a.k != L.top_k || d.a.eff != L.e_ffn) return 1;
    if (!decode_shape_ok(d.a.d, a.H, a.Hkv, a.hd, d.a.E, d.a.k, d.a.eff, L.down_q)) return 5;
    DecodeLayer &y = d.layers[(size_t)li];
    y.gain = (const int64_t *)gain.d; y.router = (const uint8_t *)r.d; y.wqkv = (const uint8_t *)wq.d; y.wo = (const uint8_t *)wo.d;
    y.tabs = L.tabs; y.kcache = kcache_dev; y.vcache = vcache_dev; y.full = full ? 1 : 0; y.down_q = L.down_q;
    if (!d.set[(size_t)li]) { d.set[(size_t)li] = true; d.n_set++; }
    d.dirty = true;
    return 0;
}

extern "C" int iie_decoder_step_dev(long long dec, int64_t *x_dev, long long pos_bound, const int *pos_dev, int *ids_out_dev,
                                    int64_t *gates_out_dev, void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!valid_decoder(dec) || !x_dev) return 1;
    DecoderObj &d = g_decoders[(size_t)dec];
    if (d.n_set != d.n_layers || pos_bound < 0 || pos_bound >= d.a.Lmax) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (d.n_ctas == 0) {
        d.n_ctas = decode_max_ctas(d.a.d, d.a.H, d.a.Hkv, d.a.hd, d.a.E, d.a.eff);
        if (d.n_ctas < d.a.Hkv) { d.n_ctas = -1; }
    }
    if (d.n_ctas < 0) return 5;
    // history keys the longest-sighted block sees at the bound: every one must fit this launch's key chunks
    bool any_full = false;
    for (const auto &y : d.layers) any_full = any_full || y.full || d.a.window <= 0;
    const long long hist = any_full ? pos_bound : std::min(pos_bound, d.a.window - 1);
    if (hist > decode_key_capacity(d.n_ctas, d.a.Hkv, d.a.hd)) return 5;
    if (!d.scratch) {
        const DecodeArgs &a = d.a;
        const size_t qkv = (size_t)(a.H + 2 * a.Hkv) * a.hd * 8, lg = (size_t)a.E * 8, gul = (size_t)a.k * 8 * a.eff;
        const size_t st = (size_t)2 * a.H * 16, acc = (size_t)2 * a.H * a.hd * 8;
        auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
        const size_t total = up(qkv) + up(lg) + up(gul) + up(st) + up(acc) + 256;
        if (cudaMalloc(&d.scratch, total) != cudaSuccess || cudaMalloc(&d.layers_dev, sizeof(DecodeLayer) * (size_t)d.n_layers) != cudaSuccess) {
            cudaGetLastError();
            if (d.scratch) { cudaFree(d.scratch); d.scratch = nullptr; }
            return 1;
        }
        uint8_t *p = d.scratch;
        d.a.qkv = (int64_t *)p; p += up(qkv);
        d.a.logits = (int64_t *)p; p += up(lg);
        d.a.gul = (int8_t *)p; p += up(gul);
        d.a.hmax = (long long *)p; d.a.Z = (unsigned long long *)(p + (size_t)2 * a.H * 8); p += up(st);
        d.a.acc = (long long *)p; p += up(acc);
        d.a.bars = (unsigned *)p;
    }
    if (d.dirty) {
        // a synchronous copy: the table must not change under a launch that is still running
        if (cudaDeviceSynchronize() != cudaSuccess ||
            cudaMemcpy(d.layers_dev, d.layers.data(), sizeof(DecodeLayer) * (size_t)d.n_layers, cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError(); return 1;
        }
        d.dirty = false;
    }
    DecodeArgs a = d.a;
    a.layers = d.layers_dev; a.x = x_dev; a.pos_bound = pos_bound; a.pos_dev = pos_dev; a.ids_out = ids_out_dev; a.gates_out = gates_out_dev;
    if (launch_decode(a, d.n_ctas, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    g_hl_d = 0;                                           // no digit planes of a single-token block are on hand any more
    return 0;
}

static void iie_decoders_drop() {
    for (auto &d : g_decoders) if (d.live) free_decoder(d);
    g_decoders.clear();
}

extern "C" void iie_decoder_destroy(long long dec) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (valid_decoder(dec)) free_decoder(g_decoders[(size_t)dec]);
}

// ====================================================================================================
// Static-scratch variant of the device-pointer product
// ====================================================================================================
// Some callers must not trigger a device allocation when they ask for a product: a serving process
// whose memory pool already owns the whole device (a cudaMalloc from a library would fail or fragment
// the pool), or a latency-critical loop that cannot afford the implicit synchronisation of
// cudaMalloc / cudaFree.  iie_apply_dev_static is iie_apply_dev with its one piece of scratch, the
// activation limb planes [T][8][K] int8, placed in the fixed array below instead of a grown workspace.
// The array is part of the library image: every GPU that loads the library holds these 4 MiB until
// the process exits.
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)4 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
static void *g_static_scratch_addr[64];        // device address of the array, per device ordinal

extern "C" int iie_apply_dev_static(long long h, const int64_t *x_dev, long long T, int fw, int64_t *out_dev,
                                    void *stream) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    // The handle was registered earlier, so the library is already initialised; nothing here allocates.
    if (g_ready != 0 || !valid_q(h) || !x_dev || !out_dev || T <= 0 || fw < 0 || fw > 62) return 1;
    const Weight &w = g_w[h];
    const long long K = w.nb * 256;
    if ((unsigned long long)T > STATIC_SCRATCH_BYTES / 8 / (unsigned long long)K) return 4;   // T*8*K bytes of limb planes
    cudaStream_t s = (cudaStream_t)stream;
    if (!fast_envelope(w.qtype, w.nb, w.maxd, w.maxdmin, fw))       // the exact 128-bit kernel needs no scratch
        return launch_exact_linear((const uint8_t *)w.d, w.qtype, w.out_f, w.nb, x_dev, T, fw, out_dev, s) == cudaSuccess ? 0 : 1;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (!g_static_scratch_addr[dev]) {
        // In host code the array's name is only a handle; the kernels need its device address.
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_static_scratch) != cudaSuccess || !addr) { cudaGetLastError(); return 1; }
        g_static_scratch_addr[dev] = addr;
    }
    int8_t *planes = (int8_t *)g_static_scratch_addr[dev];
    // Nothing in the scratch has to start at zero: the limb kernel overwrites every byte the product reads.
    if (launch_limbs(x_dev, T, K, planes, g_flags, s) != cudaSuccess) { cudaGetLastError(); return 1; }
    SkinnyArgs a = {};
    a.wa = w.cell; a.wb = w.cell; a.pairs_per_group = (int)T; a.out_f = w.out_f; a.n_blocks = w.nb; a.fw = fw; a.fa = 16;
    a.xl = planes; a.out = out_dev; a.flags = g_flags;
    if (launch_skinny(w.qtype, MODE_LINEAR, a, 1, (int)std::min<long long>(T, 4), s) != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
}
