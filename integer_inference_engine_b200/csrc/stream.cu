// Single-token ("decode") fused-dequant products: bulk-copy weight streaming into shared memory.
//
// Batch-1 decode touches each weight byte once, so the kernels are bound by HBM bandwidth and, at
// these sizes (10-14 MB per launch), by latency.  Every CTA therefore owns a contiguous run of
// 16-row tiles, asks the copy engine for ALL of its bytes up front (cp.async.bulk, one mbarrier per
// tile, nothing is recycled so no barrier is ever re-armed), and its warps unpack and multiply the
// tiles as they land.  The arithmetic is the limb-MMA scheme of skinny.cu: the activation's eight
// balanced base-256 digits are the N=8 columns of a warp MMA; sub-block scales and minimums are
// applied in int32, the block scale in int64, the columns are recombined in 128 bits and shifted
// once.  Epilogues fuse the integer SiLU * up product (gate/up pair) and the gate-weighted combine
// (down), replacing north-mini-code/tools/nmc_qk_cuda.cu:208-237 (silu_k, mul_shift_k,
// matmul_multi_k, combine_k).
//
// Column order: MMA column c carries limb (c >> 1) + 4 * (c & 1), so that when the activation needs
// at most four limbs (the usual case for normalised hidden states) every odd column is zero and
// each thread skips half of its scale multiplies.
#include <algorithm>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"
#include "norm.cuh"

namespace iie {

namespace {

constexpr int NWARPS = 16;
constexpr int FR_PAD = 32;          // padding of a digit plane in shared memory (bytes): the eight planes start on different banks
constexpr int SK_MAXK = 64, SK_MAXE = 1024;   // top-k prologue: largest k and number of logits

constexpr unsigned WAIT_LIMIT = 1u << 22;   // mbarrier polls before a wait gives up and raises flag bit 3

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the bytes never arrived (the caller raises an error flag and skips the work).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (unsigned it = 0; it < WAIT_LIMIT; it++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// floor((x << fa) / rms) in 128 bits, for rows whose values are too wide for the reciprocal path (kept out of line: rare)
__device__ __noinline__ int64_t norm_quotient_wide(int64_t xv, unsigned long long rms, int fa, bool &bad) {
    const i128 num = (i128)xv * ((i128)1 << fa);
    i128 q = num / (i128)rms;
    if (num < 0 && q * (i128)rms != num) q -= 1;
    if (q > (i128)INT64_MAX || q < (i128)INT64_MIN) { bad = true; q = 0; }
    return (int64_t)q;
}

template <int QT, int MODE, bool FAST>
__global__ void __launch_bounds__(NWARPS * 32, 1) stream_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int nb = (int)a.n_blocks;
    const long long K = a.n_blocks * 256;
    const int tile_bytes = 2 * nb * HTB;
    const int tpc = a.tiles_per_cta;
    uint8_t *wbuf = smem;
    unsigned long long *red = reinterpret_cast<unsigned long long *>(smem + (size_t)tpc * tile_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + (size_t)tpc * 128);
    int *done = reinterpret_cast<int *>(bars + tpc);             // blocks of each tile already accumulated
    int *t_sel = done + tpc, *t_pos = t_sel + tpc;               // tile -> (selected matrix slot, tile inside it)
    // MODE_FRONT only: digit planes of the normalised row [8][K + pad], the staged row and gain
    const int pstride = (int)K + FR_PAD;
    int8_t *planes = reinterpret_cast<int8_t *>((reinterpret_cast<uintptr_t>(t_pos + tpc) + 15) & ~(uintptr_t)15);
    int64_t *xs = reinterpret_cast<int64_t *>(planes + (size_t)8 * pstride);
    int64_t *gs = xs + K;
    __shared__ int s_timeout;
    __shared__ int s_ids[SK_MAXK];                               // top-k prologue: selected experts and their gates
    __shared__ long long s_gates[SK_MAXK];
    __shared__ int64_t s_lg[SK_MAXE];
    __shared__ unsigned long long s_lo[NWARPS], s_hi[NWARPS], s_mx[NWARPS], s_gmx[NWARPS];
    __shared__ unsigned long long s_rms, s_inv, s_gm;
    __shared__ int s_bad, s_nl, s_fast;

    const int n_tiles = MODE == MODE_FRONT ? a.tiles_per_expert + a.tiles_b : a.n_sel * a.tiles_per_expert;
    const int tile0 = (int)blockIdx.x * tpc;
    const int my_tiles = min(tpc, n_tiles - tile0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_ht = (int)((a.out_f + 7) >> 3), n_ht_b = (int)((a.out_f_b + 7) >> 3);
    const bool topk = MODE != MODE_FRONT && MODE != MODE_LINEAR && a.logits != nullptr;

    for (int i = threadIdx.x; i < my_tiles * 128; i += blockDim.x) red[i] = 0ULL;
    for (int i = threadIdx.x; i < my_tiles; i += blockDim.x) {
        done[i] = 0;
        const int tau = tile0 + i;
        int sl, ps;
        if (MODE == MODE_FRONT) { sl = tau < a.tiles_per_expert ? 0 : 1; ps = tau - sl * a.tiles_per_expert; }
        else { sl = tau / a.tiles_per_expert; ps = tau - sl * a.tiles_per_expert; }
        t_sel[i] = sl; t_pos[i] = ps;
        mbar_init(&bars[i], 1);
    }
    if (threadIdx.x == 0) { s_timeout = 0; s_bad = 0; s_nl = 1; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // Top-k prologue.  With early_weights the logits were final before the previous kernel started (the caller's promise,
    // as for the pointer arrays), so the ranking and the weight requests both happen before the dependency wait.
    auto rank_topk = [&]() {
        const int n = a.n_experts;
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_lg[i] = a.logits[i];
        __syncthreads();
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            const int64_t v = s_lg[e];
            int rank = 0;
            for (int j = 0; j < n; j++) { const int64_t w = s_lg[j]; rank += (w > v) || (w == v && j < e); }
            if (rank < a.n_sel) {
                const long long gt = sigmoid_fixed_c(v, a.fa, a.sig_log2e, a.sig_clip);
                s_ids[rank] = e; s_gates[rank] = gt;
                if (blockIdx.x == 0) { if (a.ids_out) a.ids_out[rank] = e; if (a.gates_out) a.gates_out[rank] = gt; }
            }
        }
        __syncthreads();
    };
    if (MODE == MODE_DOWN && a.rank_logits && my_tiles <= 0) {
        // the spare CTA: the ranking runs beside the product, on an SM the product leaves idle, instead of in the prologue of
        // every CTA of the two kernels behind this one
        const int n = a.rank_n;
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_lg[i] = a.rank_logits[i];
        __syncthreads();
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            const int64_t v = s_lg[e];
            int rank = 0;
            for (int j = 0; j < n; j++) { const int64_t w = s_lg[j]; rank += (w > v) || (w == v && j < e); }
            if (rank < a.rank_k) {
                const long long gt = sigmoid_fixed_c(v, a.fa, a.sig_log2e, a.sig_clip);
                a.rank_ids[rank] = e; a.rank_gates[rank] = gt;
                if (a.rank_tabs && a.rank_ptrs) {
#pragma unroll
                    for (int m = 0; m < 3; m++) a.rank_ptrs[m * a.rank_k + rank] = a.rank_tabs[m * n + e];
                }
                if (a.ids_out) a.ids_out[rank] = e;
                if (a.gates_out) a.gates_out[rank] = gt;
            }
        }
        return;
    }
    if (topk && a.pdl && a.early_weights) rank_topk();
    // Programmatic dependent launch: everything above touched only this CTA's shared memory.  When the
    // selected-expert pointers were final before the previous kernel started (early_weights), the weight
    // copies are requested before waiting for that kernel, so they overlap its execution.
    if (a.pdl && !a.early_weights) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }
    if (topk && !(a.pdl && a.early_weights)) rank_topk();
    // one lane per tile resolves its matrix pointer and asks the copy engine for the whole tile
    for (int i = threadIdx.x; i < my_tiles; i += blockDim.x) {
        const int s = t_sel[i], p = t_pos[i];
        const uint8_t *pa, *pb = nullptr;
        if (MODE == MODE_FRONT) pa = s == 0 ? a.wa[0] : a.wb[0];
        else if (topk) { const int e = s_ids[s]; pa = a.wa[e]; if (MODE == MODE_GATEUP) pb = a.wb[e]; }
        else if (a.sel_wa) { pa = a.sel_wa[s]; if (MODE == MODE_GATEUP) pb = a.sel_wb[s]; }
        else { const int e = a.sel ? a.sel[s] : s; pa = a.wa[e]; if (MODE == MODE_GATEUP) pb = a.wb[e]; }
        uint8_t *dst = wbuf + (size_t)i * tile_bytes;
        if (MODE == MODE_GATEUP) {
            mbar_expect_tx(&bars[i], (uint32_t)tile_bytes);
            bulk_g2s(dst, pa + (size_t)p * nb * HTB, (uint32_t)(nb * HTB), &bars[i]);
            bulk_g2s(dst + nb * HTB, pb + (size_t)p * nb * HTB, (uint32_t)(nb * HTB), &bars[i]);
        } else {
            const int units = (2 * p + 1 < ((MODE == MODE_FRONT && s == 1) ? n_ht_b : n_ht)) ? 2 : 1;   // an odd last half-tile stands alone
            mbar_expect_tx(&bars[i], (uint32_t)(units * nb * HTB));
            bulk_g2s(dst, pa + (size_t)(2 * p) * nb * HTB, (uint32_t)(units * nb * HTB), &bars[i]);
        }
    }
    if (MODE == MODE_FRONT && a.pf_base) {
        // rows the next kernel will ask for first: written by earlier steps, so they can be on their way into L2 now
        const long long pos = a.pf_pos_dev ? (long long)*a.pf_pos_dev : a.pf_pos;
        if (pos > 0 && pos <= a.pf_pos && pos < a.pf_rows && (a.pf_row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(a.pf_base) & 15) == 0) {
            const long long lo = (a.pf_window > 0 && pos - a.pf_window + 1 > 0) ? pos - a.pf_window + 1 : 0;
            const long long span = pos - lo, per_head = (span + 31) >> 5, total = per_head * a.pf_heads;
            for (long long p = blockIdx.x + (long long)gridDim.x * threadIdx.x; p < total; p += (long long)gridDim.x * blockDim.x) {
                const long long head = p / per_head, r0 = (p - head * per_head) << 5;
                const uint32_t bytes = (uint32_t)(min(32LL, span - r0) * a.pf_row_bytes);
                const char *src = reinterpret_cast<const char *>(a.pf_base) + ((head * a.pf_rows + lo + r0) * a.pf_row_bytes);
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
            }
        }
    }
    unsigned long long gmx = 0;
    if (MODE == MODE_FRONT && a.gain)                              // the gain is immutable: staged before the dependency wait
        for (int i = threadIdx.x * 2; i < (int)K; i += blockDim.x * 2) {
            const longlong2 gv = *reinterpret_cast<const longlong2 *>(a.gain + i);
            *reinterpret_cast<longlong2 *>(gs + i) = gv;
            const unsigned long long g0 = uabs64(gv.x), g1 = uabs64(gv.y);
            gmx = g0 > gmx ? g0 : gmx; gmx = g1 > gmx ? g1 : gmx;
        }
    if (a.pdl && a.early_weights) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }
    if (MODE == MODE_FRONT) {
        // ---- RMSNorm of the row and its digit planes, in every CTA (arithmetic of route.cu) ----------------------------
        u128 ssq = 0; unsigned long long mx = 0;
        for (int i = threadIdx.x * 2; i < (int)K; i += blockDim.x * 4) {          // two loads in flight per thread
            const int i2 = i + blockDim.x * 2;
            const longlong2 xv = *reinterpret_cast<const longlong2 *>(a.x + i);
            longlong2 xw = make_longlong2(0, 0);
            if (i2 < (int)K) xw = *reinterpret_cast<const longlong2 *>(a.x + i2);
            *reinterpret_cast<longlong2 *>(xs + i) = xv;
            if (i2 < (int)K) *reinterpret_cast<longlong2 *>(xs + i2) = xw;
            const unsigned long long v0 = uabs64(xv.x), v1 = uabs64(xv.y), v2 = uabs64(xw.x), v3 = uabs64(xw.y);
            ssq += (u128)v0 * v0; ssq += (u128)v1 * v1; ssq += (u128)v2 * v2; ssq += (u128)v3 * v3;
            mx = v0 > mx ? v0 : mx; mx = v1 > mx ? v1 : mx; mx = v2 > mx ? v2 : mx; mx = v3 > mx ? v3 : mx;
        }
        unsigned long long lo = (unsigned long long)ssq, hi = (unsigned long long)(ssq >> 64);
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) {
            const unsigned long long lo2 = __shfl_xor_sync(0xffffffffu, lo, sft), hi2 = __shfl_xor_sync(0xffffffffu, hi, sft);
            const u128 sum = (((u128)hi << 64) | lo) + (((u128)hi2 << 64) | lo2);
            lo = (unsigned long long)sum; hi = (unsigned long long)(sum >> 64);
            const unsigned long long m2 = __shfl_xor_sync(0xffffffffu, mx, sft), g2 = __shfl_xor_sync(0xffffffffu, gmx, sft);
            mx = m2 > mx ? m2 : mx; gmx = g2 > gmx ? g2 : gmx;
        }
        if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; s_mx[warp] = mx; s_gmx[warp] = gmx; }
        __syncthreads();
        if (warp == 0) {
            lo = lane < NWARPS ? s_lo[lane] : 0ULL; hi = lane < NWARPS ? s_hi[lane] : 0ULL;
            mx = lane < NWARPS ? s_mx[lane] : 0ULL; gmx = lane < NWARPS ? s_gmx[lane] : 0ULL;
#pragma unroll
            for (int sft = NWARPS / 2; sft > 0; sft >>= 1) {
                const unsigned long long lo2 = __shfl_xor_sync(0xffffffffu, lo, sft), hi2 = __shfl_xor_sync(0xffffffffu, hi, sft);
                const u128 sum = (((u128)hi << 64) | lo) + (((u128)hi2 << 64) | lo2);
                lo = (unsigned long long)sum; hi = (unsigned long long)(sum >> 64);
                const unsigned long long m2 = __shfl_xor_sync(0xffffffffu, mx, sft), g2 = __shfl_xor_sync(0xffffffffu, gmx, sft);
                mx = m2 > mx ? m2 : mx; gmx = g2 > gmx ? g2 : gmx;
            }
        }
        if (threadIdx.x == 0) {
            const u128 total = ((u128)hi << 64) | lo;
            const unsigned long long m = mx, gm = gmx;
            int bad = m > (1ULL << 57) ? 1 : 0;                  // keeps the 128-bit sum of squares exact
            const int d = (int)K;
            u128 mean;
            if ((d & (d - 1)) == 0) mean = total >> (31 - __clz(d));
            else if ((total >> 64) == 0) mean = (u128)((unsigned long long)total / (unsigned long long)d);
            else mean = total / (u128)(unsigned long long)d;
            const u128 rms = isqrt128(mean + a.eps);
            if (rms == 0 || rms > (u128)0xFFFFFFFFFFFFFFFFULL) bad = 1;
            s_rms = (unsigned long long)rms; s_gm = gm; s_bad = bad;
            const unsigned long long inv = recip_below((unsigned long long)rms);
            s_inv = inv;
            // block-wide bound: with q <= n / rms + 1 for every quotient and |gain| <= gm, n < rms * (2^31 - 2) keeps the
            // quotients in 32 bits and n * gm <= rms * ((L - 2) * 2^fa - gm) keeps every gain product within the four-digit
            // range L = 0x7F7F7F7F; the per-element range tests then drop out of the loop below
            bool fast = false;
            if (!bad && a.gain && a.fa <= 30 && m < (1ULL << (62 - a.fa)) && rms < ((u128)1 << 62) && gm < (1ULL << 31)) {
                const unsigned long long n = m << a.fa, r64 = (unsigned long long)rms, lim = 2139062141ULL << a.fa;
                fast = (u128)n < (u128)r64 * 2147483646ULL && lim > gm && (u128)n * gm <= (u128)r64 * (lim - gm);
            }
            s_fast = fast ? 1 : 0;
        }
        __syncthreads();
        const unsigned long long rms = s_rms, inv = s_inv, gm = s_gm;
        const bool dead = s_bad != 0;                             // not normalisable exactly: flag raised, zero planes, the launch still drains its copies
        bool bad = false, over = false;
        int nl = 1;
        if (s_fast) {
            const int fa = a.fa;
            for (int i = threadIdx.x * 4; i < (int)K; i += blockDim.x * 4) {
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int64_t xv = xs[i + e];
                    const unsigned long long n = uabs64(xv) << fa;
                    unsigned long long q = __umul64hi(n, inv), r = n - q * rms;
                    while (r >= rms) { q++; r -= rms; }
                    const int yq = xv >= 0 ? (int)q : -(int)q - (r != 0);                      // floor of the signed quotient
                    const int64_t y = ((int64_t)yq * (int)gs[i + e]) >> fa;                    // both factors fit 32 bits here
                    pk[e] = ((uint32_t)(int)y + 0x80808080u) ^ 0x80808080u;                    // byte l = balanced digit l
                }
                const uint32_t any = pk[0] | pk[1] | pk[2] | pk[3];
                nl = max(nl, any == 0 ? 1 : 4 - (__clz((int)any) >> 3));
                const uint32_t lo01 = __byte_perm(pk[0], pk[1], 0x5140), hi01 = __byte_perm(pk[0], pk[1], 0x7362);
                const uint32_t lo23 = __byte_perm(pk[2], pk[3], 0x5140), hi23 = __byte_perm(pk[2], pk[3], 0x7362);
                uint32_t pw[8] = {__byte_perm(lo01, lo23, 0x5410), __byte_perm(lo01, lo23, 0x7632),
                                  __byte_perm(hi01, hi23, 0x5410), __byte_perm(hi01, hi23, 0x7632), 0, 0, 0, 0};
#pragma unroll
                for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * pstride + i) = pw[l];
                if (blockIdx.x == 0 && a.hl_out) {
#pragma unroll
                    for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(a.hl_out + (long long)l * K + i) = pw[l];
                }
            }
        } else
        for (int i = threadIdx.x * 4; i < (int)K; i += blockDim.x * 4) {
            uint32_t pw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int64_t xv = xs[i + e];
                int64_t y = xv;
                bool small = false;
                if (dead) y = 0;
                else if (a.gain) {
                    if (uabs64(xv) < (1ULL << (62 - a.fa)) && rms < (1ULL << 62)) {
                        y = floor_div_recip(xv * ((long long)1 << a.fa), rms, inv);
                        small = uabs64(y) < (1ULL << 31) && gm < (1ULL << 31);
                    } else y = norm_quotient_wide(xv, rms, a.fa, bad);
                    if (small) y = (y * gs[i + e]) >> a.fa;                       // |y * gain| < 2^62: the 64-bit product is exact
                    else {
                        if ((u128)uabs64(y) * gm > (u128)INT64_MAX) bad = true;  // the oracle refuses such a gain product
                        y = mul_shift(y, gs[i + e], a.fa);
                    }
                }
                if (y >= -2147483648LL && y <= 2139062143LL) {
                    // four balanced digits hold it: 32-bit arithmetic, the upper planes stay zero
                    const uint32_t pk = ((uint32_t)(int)y + 0x80808080u) ^ 0x80808080u;      // byte l = balanced digit l (the sum cannot wrap in this range)
                    nl = max(nl, pk == 0 ? 1 : 4 - (__clz((int)pk) >> 3));
#pragma unroll
                    for (int l = 0; l < 4; l++) pw[l] |= ((pk >> (8 * l)) & 0xFF) << (8 * e);
                } else {
                    bool ok;
                    const uint64_t dg = balanced_digits8(y, ok);
                    over |= !ok;
                    nl = max(nl, digits_used(dg));
#pragma unroll
                    for (int l = 0; l < 8; l++) pw[l] |= (uint32_t)((dg >> (8 * l)) & 0xFF) << (8 * e);
                }
            }
#pragma unroll
            for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * pstride + i) = pw[l];
            if (blockIdx.x == 0 && a.hl_out) {
#pragma unroll
                for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(a.hl_out + (long long)l * K + i) = pw[l];
            }
        }
        if ((bad || dead) && lane == 0) atomicOr(a.flags, 2);
        if (over) atomicOr(a.flags, 1);
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4));  nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
        if (lane == 0) atomicMax(&s_nl, nl);
        __syncthreads();
        if (blockIdx.x == 0 && threadIdx.x == 0) { if (a.h_nl_out) *a.h_nl_out = s_nl; if (a.gu_nl_zero) *a.gu_nl_zero = 0; }
    }
    int x_digits = 8;
    if (MODE == MODE_FRONT) x_digits = s_nl;
    else if (a.x_nl) {                                           // a producer may leave one count per part of the row
        x_digits = a.x_nl[0];
        for (int i = 1; i < a.x_nl_n; i++) x_digits = max(x_digits, a.x_nl[i]);
    }
    const bool half = x_digits <= 4;

    // items (tile, block) are dealt round-robin to the warps; indices advance without divisions
    const int n_items = my_tiles * nb;
    const int step_t = NWARPS / nb, step_b = NWARPS - step_t * nb;
    int ti = warp / nb, b = warp - ti * nb;
    const int g = lane >> 2, t = lane & 3;
    const long long xoff = (long long)col_limb(g) * K;
    uint32_t bf[16];
    const int8_t *xcur = nullptr;
    int bcur = -1;
    for (int it = warp; it < n_items; it += NWARPS) {
        const int s = t_sel[ti], p = t_pos[ti];
        const int8_t *xp = MODE == MODE_FRONT ? planes : a.xl + (a.x_per_sel ? (long long)s * 8 * K : 0);
        if (xp != xcur || b != bcur) {                        // activation fragments: reused while (vector, block) repeat
            if (MODE == MODE_FRONT) load_bfrag<QT, false>(planes + col_limb(g) * pstride + b * 256, t, bf);
            else load_bfrag<QT, true>(xp + xoff + (long long)b * 256, t, bf);
            xcur = xp; bcur = b;
        }
        const uint8_t *ua = wbuf + (size_t)ti * tile_bytes + (size_t)b * HTB;
        const uint8_t *ub;
        if (MODE == MODE_GATEUP) ub = ua + (size_t)nb * HTB;
        else ub = (2 * p + 1 < ((MODE == MODE_FRONT && s == 1) ? n_ht_b : n_ht)) ? ua + (size_t)nb * HTB : ua;
        const int ti_now = ti;
        b += step_b; ti += step_t;
        if (b >= nb) { b -= nb; ti++; }
        if (!mbar_wait(&bars[ti_now], 0)) { s_timeout = 1; continue; }
        int64_t acc[4] = {0, 0, 0, 0};
        run_item<QT, FAST>(ua, ub, lane, a.fw, bf, half, acc);
        unsigned long long *r = red + (size_t)ti_now * 128;
        atomicAdd(&r[g * 8 + 2 * t], (unsigned long long)acc[0]);
        atomicAdd(&r[(g + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
        if (!half) {
            atomicAdd(&r[g * 8 + 2 * t + 1], (unsigned long long)acc[1]);
            atomicAdd(&r[(g + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
        }
        if (MODE == MODE_GATEUP) continue;                    // its epilogue is long: all rows run it in parallel below
        // the warp that completes a tile (all nb blocks added) runs its epilogue; nobody waits
        __threadfence_block();
        int prior = 0;
        if (lane == 0) prior = atomicAdd(&done[ti_now], 1);
        prior = __shfl_sync(0xffffffffu, prior, 0);
        if (prior != nb - 1) continue;
        __threadfence_block();
        const volatile unsigned long long *rv = r;
        if (lane < 16) {
            const long long row = (long long)p * 16 + lane;
            if (row < ((MODE == MODE_FRONT && s == 1) ? a.out_f_b : a.out_f)) {
                unsigned long long cc[8];
#pragma unroll
                for (int c = 0; c < 8; c++) cc[c] = rv[lane * 8 + c];
                const int64_t y = recombine_cols(cc, a.fw);
                if (MODE == MODE_FRONT) (s == 0 ? a.out : a.out_b)[row] = y;
                else if (MODE == MODE_LINEAR) a.out[(long long)s * a.out_f + row] = y;
                else atomicAdd(reinterpret_cast<unsigned long long *>(a.out + row),
                               (unsigned long long)mul_shift(y, topk ? s_gates[s] : a.gates[s], a.fa));
            }
        }
    }
    if (MODE == MODE_GATEUP) {
        // rows 0..7 of a tile are the gate projection, rows 8..15 the up projection of the same output index
        __syncthreads();
        int nl = 0;
        for (int idx = threadIdx.x; idx < my_tiles * 8; idx += blockDim.x) {
            const int tq = idx >> 3, r8 = idx & 7;
            const int s = t_sel[tq], p = t_pos[tq];
            const long long row = (long long)p * 8 + r8;
            if (row >= a.out_f) continue;
            const unsigned long long *rr = red + (size_t)tq * 128;
            const int64_t yg = recombine_cols(rr + r8 * 8, a.fw), yu = recombine_cols(rr + (r8 + 8) * 8, a.fw);
            const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
            const int64_t gu = mul_shift(sg, yu, a.fa);
            if (a.out) a.out[(long long)s * a.out_f + row] = gu;
            bool ok;
            const uint64_t d = balanced_digits8(gu, ok);
            if (!ok) atomicOr(a.flags, 1);
            nl = max(nl, digits_used(d));
#pragma unroll
            for (int l = 0; l < 8; l++) a.out_limbs[((long long)s * 8 + l) * a.out_f + row] = (int8_t)(d >> (8 * l));
        }
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4));  nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
        if (lane == 0 && nl > 0 && a.out_nl) atomicMax(a.out_nl, nl);
    }
    __syncthreads();
    if (s_timeout && threadIdx.x == 0) atomicOr(a.flags, 8);
}

template <int QT, int MODE, bool FAST>
cudaError_t launch_stream_t(const StreamArgs &a_in, cudaStream_t s) {
    StreamArgs a = a_in;
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const long long n_ht = (a.out_f + 7) >> 3;
    a.tiles_per_expert = (int)(MODE == MODE_GATEUP ? n_ht : (n_ht + 1) / 2);
    a.tiles_b = MODE == MODE_FRONT ? (int)((((a.out_f_b + 7) >> 3) + 1) / 2) : 0;
    const long long n_tiles = MODE == MODE_FRONT ? (long long)a.tiles_per_expert + a.tiles_b : (long long)a.n_sel * a.tiles_per_expert;
    const size_t tile_bytes = (size_t)2 * a.n_blocks * HTB, per_tile = tile_bytes + 128 * 8 + 8 + 12;
    const size_t front_bytes = MODE == MODE_FRONT ? (size_t)8 * (a.n_blocks * 256 + FR_PAD) + (size_t)16 * a.n_blocks * 256 + 16 : 0;
    if (MODE == MODE_FRONT && (!a.x || !a.out || !a.out_b || a.out_f_b <= 0 || a.n_blocks * 256 > 8192)) return cudaErrorInvalidValue;
    if (MODE != MODE_FRONT && a.logits && (a.n_experts <= 0 || a.n_experts > SK_MAXE || a.n_sel > SK_MAXK || a.n_sel > a.n_experts)) return cudaErrorInvalidValue;
    const int max_tpc = (int)((200 * 1024 - front_bytes) / per_tile);
    if (max_tpc < 1) return cudaErrorInvalidConfiguration;
    int tpc = (int)((n_tiles + 147) / 148);                      // one wave when everything fits
    if (tpc > max_tpc) tpc = max_tpc;                            // several waves: one CTA per SM (registers), so the longest run that fits
    a.tiles_per_cta = tpc;
    a.sig_log2e = sigmoid_log2e(a.fa); a.sig_clip = sigmoid_clip(a.fa);
    if (a.rank_logits && (MODE != MODE_DOWN || a.rank_n <= 0 || a.rank_n > SK_MAXE || a.rank_k <= 0 || a.rank_k > a.rank_n || !a.rank_ids || !a.rank_gates))
        return cudaErrorInvalidValue;
    const unsigned grid = (unsigned)((n_tiles + tpc - 1) / tpc) + (a.rank_logits ? 1u : 0u);   // + the CTA that only ranks
    const size_t smem = (size_t)tpc * per_tile + 64 + front_bytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(stream_kernel<QT, MODE, FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 214 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NWARPS * 32); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = a.pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, stream_kernel<QT, MODE, FAST>, a);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <int QT, int MODE>
cudaError_t launch_stream_f(const StreamArgs &a, cudaStream_t s) {
    return a.fast ? launch_stream_t<QT, MODE, true>(a, s) : launch_stream_t<QT, MODE, false>(a, s);
}

}  // namespace

cudaError_t launch_stream(int qtype, int mode, const StreamArgs &a, cudaStream_t s) {
    if (a.n_sel <= 0 || a.out_f <= 0 || a.n_blocks <= 0) return cudaErrorInvalidValue;
    if (qtype == QT_Q4K) {
        if (mode == MODE_LINEAR) return launch_stream_f<QT_Q4K, MODE_LINEAR>(a, s);
        if (mode == MODE_GATEUP) return launch_stream_f<QT_Q4K, MODE_GATEUP>(a, s);
        if (mode == MODE_FRONT) return launch_stream_f<QT_Q4K, MODE_FRONT>(a, s);
        return launch_stream_f<QT_Q4K, MODE_DOWN>(a, s);
    }
    if (qtype == QT_Q6K) {
        if (mode == MODE_LINEAR) return launch_stream_f<QT_Q6K, MODE_LINEAR>(a, s);
        if (mode == MODE_GATEUP) return launch_stream_f<QT_Q6K, MODE_GATEUP>(a, s);
        if (mode == MODE_FRONT) return launch_stream_f<QT_Q6K, MODE_FRONT>(a, s);
        return launch_stream_f<QT_Q6K, MODE_DOWN>(a, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace iie
