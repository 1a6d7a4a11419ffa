// Single-token routing + gate/up in ONE launch.
//
// The routing of a token (RMSNorm, digit planes, 128 router rows, top-k, sigmoid gates) is a few microseconds
// of dependent latency and 147 KB of weights; run as its own launch it costs as much as the gate/up product it
// precedes.  Here EVERY CTA of the gate/up grid recomputes the routing for itself:
//   * before the dependency wait each CTA asks the copy engine for the whole router (the bytes do not depend
//     on the token) into the shared-memory buffer that later holds its expert tiles, and stages the norm gain;
//   * after the wait: stage x, 128-bit sum of squares, exact isqrt, reciprocal floor division, gain, balanced
//     digits -> planes in shared memory; router rows as (tile, block) items over the warps; logits; rank-based
//     top-k (greater value first, lower index on ties); sigmoid gates;
//   * the CTA then knows which experts were selected without any global round trip, requests its own run of
//     gate/up tiles of those experts into the (now free) router buffer and proceeds exactly like the streamed
//     gate/up kernel: K-split warps, shared-memory reduction, SiLU * up epilogue, digit planes of gu.
// CTA 0 also publishes ids, gates and the selected down-projection pointers for the down launch and
// initialises the block's output row.  Arithmetic and envelope flags are those of route.cu and stream.cu
// (north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72, cohere2.py:162-188).
// Redundant work per CTA: ~2 us; saved: one launch, one grid drain and the pointer round trip per block.
#include <algorithm>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"

namespace iie {

namespace {

constexpr int RG_WARPS = 16, RG_THREADS = RG_WARPS * 32;
constexpr int RG_PAD = 32;                 // plane padding (bytes): keeps the 8 digit planes on different banks
constexpr unsigned RG_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ unsigned long long rg_uabs(int64_t v) { return v < 0 ? (0ULL - (unsigned long long)v) : (unsigned long long)v; }

__device__ u128 rg_isqrt128(u128 v) {
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

// floor(num / den) for |num| < 2^62 and 0 < den < 2^62 through inv = floor((2^64 - 1) / den)
__device__ __forceinline__ int64_t rg_floor_div(int64_t num, unsigned long long den, unsigned long long inv) {
    const unsigned long long n = rg_uabs(num);
    unsigned long long q = __umul64hi(n, inv), r = n - q * den;
    while (r >= den) { q++; r -= den; }
    return num >= 0 ? (int64_t)q : -(int64_t)q - (r != 0);
}

__device__ __forceinline__ uint32_t rg_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rg_bar_init(uint64_t *bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rg_u32(bar))); }
__device__ __forceinline__ void rg_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rg_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rg_wait(uint64_t *bar) {
    for (unsigned it = 0; it < RG_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(rg_u32(bar)) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void rg_bulk(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(rg_u32(dst)), "l"(src), "r"(bytes), "r"(rg_u32(bar)) : "memory");
}

struct RgLayout { int wbuf, planes, xs, gs, red_r, red_t, logits, ids, gates, bars_r, bars_t, total; };

__host__ __device__ inline RgLayout rg_layout(int d, int n_rt, int tpc, int tile_bytes, int n_experts, int k) {
    RgLayout L;
    int o = 0;
    L.wbuf = o; o += (n_rt > tpc ? n_rt : tpc) * tile_bytes;
    o = (o + 127) & ~127;
    L.planes = o; o += 8 * (d + RG_PAD);
    L.xs = o; o += 8 * d;
    L.gs = o; o += 8 * d;
    L.red_r = o; o += n_rt * 1024;
    L.red_t = o; o += tpc * 1024;
    L.logits = o; o += 8 * ((n_experts + 15) & ~15);
    L.gates = o; o += 8 * k;
    L.ids = o; o += 4 * ((k + 1) & ~1);
    L.bars_r = o; o += 8 * n_rt;
    L.bars_t = o; o += 8 * tpc;
    L.total = o;
    return L;
}

template <int QT, bool FAST>
__global__ void __launch_bounds__(RG_THREADS, 1) routed_gateup_kernel(const RoutedGateUpArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int d = a.d, stride = d + RG_PAD, nb = d / 256, tile_bytes = 2 * nb * HTB;
    const int n = a.n_experts, k = a.k, tpc = a.tiles_per_cta;
    const int n_hr = (n + 7) >> 3, n_rt = (n_hr + 1) >> 1;               // router half-tiles / 16-row tiles
    const RgLayout L = rg_layout(d, n_rt, tpc, tile_bytes, n, k);
    uint8_t *wbuf = smem + L.wbuf;
    int8_t *planes = reinterpret_cast<int8_t *>(smem + L.planes);
    int64_t *xs = reinterpret_cast<int64_t *>(smem + L.xs), *gs = reinterpret_cast<int64_t *>(smem + L.gs);
    unsigned long long *red_r = reinterpret_cast<unsigned long long *>(smem + L.red_r);
    unsigned long long *red_t = reinterpret_cast<unsigned long long *>(smem + L.red_t);
    int64_t *s_logits = reinterpret_cast<int64_t *>(smem + L.logits), *s_gates = reinterpret_cast<int64_t *>(smem + L.gates);
    int *s_ids = reinterpret_cast<int *>(smem + L.ids);
    uint64_t *bars_r = reinterpret_cast<uint64_t *>(smem + L.bars_r), *bars_t = reinterpret_cast<uint64_t *>(smem + L.bars_t);
    __shared__ unsigned long long s_lo[RG_WARPS], s_hi[RG_WARPS], s_max[RG_WARPS], s_gmax[RG_WARPS];
    __shared__ unsigned long long s_rms, s_inv, s_gm;
    __shared__ int s_bad, s_nl, s_timeout;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    const int n_tiles = k * a.tiles_per_expert;
    const int tile0 = (int)blockIdx.x * tpc, my_tiles = max(0, min(tpc, n_tiles - tile0));

    // ---- before the dependency wait: only immutable data and this CTA's shared memory ---------------------------
    if (tid == 0) { s_bad = 0; s_nl = 1; s_timeout = 0; }
    for (int i = tid; i < n_rt; i += RG_THREADS) rg_bar_init(&bars_r[i]);
    for (int i = tid; i < tpc; i += RG_THREADS) rg_bar_init(&bars_t[i]);
    for (int i = tid; i < (n_rt + tpc) * 128; i += RG_THREADS) red_r[i] = 0ULL;       // red_r and red_t are contiguous
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    if (tid < n_rt) {
        const int units = (2 * tid + 1 < n_hr) ? 2 : 1;
        rg_expect(&bars_r[tid], (uint32_t)(units * nb * HTB));
        rg_bulk(wbuf + (size_t)tid * tile_bytes, a.router + (size_t)(2 * tid) * nb * HTB, (uint32_t)(units * nb * HTB), &bars_r[tid]);
    }
    unsigned long long gmx = 0;
    if (a.gain)
        for (int i = tid * 2; i < d; i += RG_THREADS * 2) {
            const longlong2 gv = *reinterpret_cast<const longlong2 *>(a.gain + i);
            *reinterpret_cast<longlong2 *>(gs + i) = gv;
            const unsigned long long g0 = rg_uabs(gv.x), g1 = rg_uabs(gv.y);
            gmx = g0 > gmx ? g0 : gmx; gmx = g1 > gmx ? g1 : gmx;
        }
    if (a.pdl) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }

    // ---- stage x, sum of squares and magnitudes ------------------------------------------------------------------
    {
        u128 ssq = 0; unsigned long long mx = 0;
        for (int i = tid * 2; i < d; i += RG_THREADS * 2) {
            const longlong2 xv = *reinterpret_cast<const longlong2 *>(a.x + i);
            *reinterpret_cast<longlong2 *>(xs + i) = xv;
            const unsigned long long v0 = rg_uabs(xv.x), v1 = rg_uabs(xv.y);
            ssq += (u128)v0 * v0; ssq += (u128)v1 * v1;
            mx = v0 > mx ? v0 : mx; mx = v1 > mx ? v1 : mx;
        }
        if (a.gain) {
            unsigned long long lo = (unsigned long long)ssq, hi = (unsigned long long)(ssq >> 64);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                const unsigned long long lo2 = __shfl_xor_sync(0xffffffffu, lo, s), hi2 = __shfl_xor_sync(0xffffffffu, hi, s);
                const u128 sum = (((u128)hi << 64) | lo) + (((u128)hi2 << 64) | lo2);
                lo = (unsigned long long)sum; hi = (unsigned long long)(sum >> 64);
                const unsigned long long m2 = __shfl_xor_sync(0xffffffffu, mx, s), g2 = __shfl_xor_sync(0xffffffffu, gmx, s);
                mx = m2 > mx ? m2 : mx; gmx = g2 > gmx ? g2 : gmx;
            }
            if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; s_max[warp] = mx; s_gmax[warp] = gmx; }
            __syncthreads();
            if (tid == 0) {
                u128 total = 0; unsigned long long m = 0, gm = 0;
                for (int i = 0; i < RG_WARPS; i++) {
                    total += ((u128)s_hi[i] << 64) | s_lo[i];
                    m = s_max[i] > m ? s_max[i] : m; gm = s_gmax[i] > gm ? s_gmax[i] : gm;
                }
                if (m > (1ULL << 57)) s_bad = 1;                 // keeps the 128-bit sum of squares exact
                u128 mean;
                if ((total >> 64) == 0) mean = (u128)((unsigned long long)total / (unsigned long long)d);
                else mean = total / (u128)(unsigned long long)d;
                const u128 rms = rg_isqrt128(mean + a.eps);
                if (rms == 0 || rms > (u128)0xFFFFFFFFFFFFFFFFULL) s_bad = 1;
                s_rms = (unsigned long long)rms; s_gm = gm;
                s_inv = rms != 0 ? 0xFFFFFFFFFFFFFFFFULL / (unsigned long long)rms : 0;
            }
        }
    }
    __syncthreads();
    if (s_bad) {                                                 // uniform over the grid; the router copies must land before exit
        if (tid == 0 && blockIdx.x == 0) atomicOr(a.flags, 2);
        if (tid < n_rt) rg_wait(&bars_r[tid]);
        return;
    }

    // ---- normalise, apply the gain, split into digit planes (four consecutive elements per step) ---------------------
    {
        const unsigned long long rms = s_rms, inv = s_inv, gm = s_gm;
        bool bad = false, over = false;
        int nl = 1;
        for (int i = tid * 4; i < d; i += RG_THREADS * 4) {
            uint32_t pw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int64_t xv = xs[i + e];
                int64_t y = xv;
                if (a.gain) {
                    if (rg_uabs(xv) < (1ULL << (62 - a.fa)) && rms < (1ULL << 62)) y = rg_floor_div(xv * ((long long)1 << a.fa), rms, inv);
                    else {
                        const i128 num = (i128)xv * ((i128)1 << a.fa);
                        i128 q = num / (i128)rms;
                        if (num < 0 && q * (i128)rms != num) q -= 1;
                        if (q > (i128)INT64_MAX || q < (i128)INT64_MIN) { bad = true; q = 0; }
                        y = (int64_t)q;
                    }
                    if ((u128)rg_uabs(y) * gm > (u128)INT64_MAX) bad = true;      // the oracle refuses such a gain product
                    y = mul_shift(y, gs[i + e], a.fa);
                }
                bool ok;
                const uint64_t dg = balanced_digits8(y, ok);
                over |= !ok;
                nl = max(nl, digits_used(dg));
#pragma unroll
                for (int l = 0; l < 8; l++) pw[l] |= (uint32_t)((dg >> (8 * l)) & 0xFF) << (8 * e);
            }
#pragma unroll
            for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * stride + i) = pw[l];
            if (blockIdx.x == 0 && a.init_out && a.init_mode)
                for (int e = 0; e < 4; e++) a.init_out[i + e] = a.init_mode == 2 ? xs[i + e] : 0;
        }
        if (blockIdx.x == 0) { if (bad) atomicOr(a.flags, 2); if (over) atomicOr(a.flags, 1); }
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4));  nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
        if (lane == 0) atomicMax(&s_nl, nl);
    }
    __syncthreads();
    const bool half = s_nl <= 4;
    if (blockIdx.x == 0 && tid == 0 && a.gu_nl_next) *a.gu_nl_next = 0;     // the cell the NEXT block's launch will use

    // ---- router rows: (tile, block) items over the warps -------------------------------------------------------------
    {
        uint32_t bf[16];
        int bcur = -1;
        const int n_items = n_rt * nb;
        for (int it = warp; it < n_items; it += RG_WARPS) {
            const int ti = it / nb, b = it - ti * nb;
            if (b != bcur) { load_bfrag<QT, false>(planes + col_limb(g) * stride + b * 256, t, bf); bcur = b; }
            const uint8_t *ua = wbuf + (size_t)ti * tile_bytes + (size_t)b * HTB;
            const uint8_t *ub = (2 * ti + 1 < n_hr) ? ua + (size_t)nb * HTB : ua;
            if (!rg_wait(&bars_r[ti])) { s_timeout = 1; continue; }
            int64_t acc[4] = {0, 0, 0, 0};
            run_item<QT, false>(ua, ub, lane, a.fw, bf, half, acc);
            unsigned long long *r = red_r + (size_t)ti * 128;
            atomicAdd(&r[g * 8 + 2 * t], (unsigned long long)acc[0]);
            atomicAdd(&r[(g + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
            if (!half) {
                atomicAdd(&r[g * 8 + 2 * t + 1], (unsigned long long)acc[1]);
                atomicAdd(&r[(g + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
            }
        }
    }
    __syncthreads();                                             // all router tiles read: their buffer is free
    for (int row = tid; row < n; row += RG_THREADS) s_logits[row] = recombine_cols(red_r + (size_t)(row >> 4) * 128 + (row & 15) * 8, a.fw);
    __syncthreads();
    // ---- top-k by rank: four lanes share one expert's comparisons -----------------------------------------------------
    {
        const int64_t log2e = sigmoid_log2e(a.fa), clip = sigmoid_clip(a.fa);
        const int part = tid & 3, per = (n + 3) >> 2, j0 = min(n, part * per), j1 = min(n, j0 + per);
        for (int e0 = 0; e0 < n; e0 += RG_THREADS / 4) {
            const int e = e0 + (tid >> 2);
            const bool live = e < n;
            const int64_t v = live ? s_logits[e] : 0;
            int rank = 0;
            if (live)
                for (int j = j0; j < j1; j++) { const int64_t w = s_logits[j]; rank += (w > v) || (w == v && j < e); }
            rank += __shfl_xor_sync(0xffffffffu, rank, 2); rank += __shfl_xor_sync(0xffffffffu, rank, 1);
            if (live && part == 0 && rank < k) { s_ids[rank] = e; s_gates[rank] = sigmoid_fixed_c(v, a.fa, log2e, clip); }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic reads of the router tiles before async writes
    __syncthreads();
    if (blockIdx.x == 0 && tid < k) {
        a.ids[tid] = s_ids[tid]; a.gates[tid] = s_gates[tid];
        a.sel_down[tid] = a.tabs[(size_t)2 * n + s_ids[tid]];
    }

    // ---- this CTA's gate/up tiles of the selected experts ------------------------------------------------------------
    if (tid < my_tiles) {
        const int tau = tile0 + tid, sl = tau / a.tiles_per_expert, p = tau - sl * a.tiles_per_expert, e = s_ids[sl];
        const uint8_t *pa = a.tabs[e], *pb = a.tabs[(size_t)n + e];
        uint8_t *dst = wbuf + (size_t)tid * tile_bytes;
        rg_expect(&bars_t[tid], (uint32_t)tile_bytes);
        rg_bulk(dst, pa + (size_t)p * nb * HTB, (uint32_t)(nb * HTB), &bars_t[tid]);
        rg_bulk(dst + nb * HTB, pb + (size_t)p * nb * HTB, (uint32_t)(nb * HTB), &bars_t[tid]);
    }
    {
        uint32_t bf[16];
        int bcur = -1;
        const int n_items = my_tiles * nb;
        for (int it = warp; it < n_items; it += RG_WARPS) {
            const int ti = it / nb, b = it - ti * nb;
            if (b != bcur) { load_bfrag<QT, false>(planes + col_limb(g) * stride + b * 256, t, bf); bcur = b; }
            const uint8_t *ua = wbuf + (size_t)ti * tile_bytes + (size_t)b * HTB, *ub = ua + (size_t)nb * HTB;
            if (!rg_wait(&bars_t[ti])) { s_timeout = 1; continue; }
            int64_t acc[4] = {0, 0, 0, 0};
            run_item<QT, FAST>(ua, ub, lane, a.fw, bf, half, acc);
            unsigned long long *r = red_t + (size_t)ti * 128;
            atomicAdd(&r[g * 8 + 2 * t], (unsigned long long)acc[0]);
            atomicAdd(&r[(g + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
            if (!half) {
                atomicAdd(&r[g * 8 + 2 * t + 1], (unsigned long long)acc[1]);
                atomicAdd(&r[(g + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
            }
        }
    }
    __syncthreads();
    // ---- epilogue: rows 0..7 of a tile are the gate projection, rows 8..15 the up projection of the same index ------
    {
        int nl = 0;
        for (int idx = tid; idx < my_tiles * 8; idx += RG_THREADS) {
            const int tq = idx >> 3, r8 = idx & 7;
            const int tau = tile0 + tq, sl = tau / a.tiles_per_expert, p = tau - sl * a.tiles_per_expert;
            const long long row = (long long)p * 8 + r8;
            if (row >= a.e_ffn) continue;
            const unsigned long long *rr = red_t + (size_t)tq * 128;
            const int64_t yg = recombine_cols(rr + r8 * 8, a.fw), yu = recombine_cols(rr + (r8 + 8) * 8, a.fw);
            const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
            const int64_t gu = mul_shift(sg, yu, a.fa);
            bool ok;
            const uint64_t dg = balanced_digits8(gu, ok);
            if (!ok) atomicOr(a.flags, 1);
            nl = max(nl, digits_used(dg));
#pragma unroll
            for (int l = 0; l < 8; l++) a.out_limbs[((long long)sl * 8 + l) * a.e_ffn + row] = (int8_t)(dg >> (8 * l));
        }
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4));  nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
        if (lane == 0 && nl > 0) atomicMax(a.gu_nl, nl);
    }
    __syncthreads();
    if (s_timeout && tid == 0) atomicOr(a.flags, 8);
}

template <int QT, bool FAST>
cudaError_t launch_t(const RoutedGateUpArgs &a_in, cudaStream_t s) {
    RoutedGateUpArgs a = a_in;
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int nb = a.d / 256, tile_bytes = 2 * nb * HTB;
    const int n_rt = (((a.n_experts + 7) >> 3) + 1) >> 1;
    a.tiles_per_expert = (int)((a.e_ffn + 7) >> 3);
    const long long n_tiles = (long long)a.k * a.tiles_per_expert;
    int tpc = (int)((n_tiles + 147) / 148);
    RgLayout L = rg_layout(a.d, n_rt, tpc, tile_bytes, a.n_experts, a.k);
    if (L.total > 225 * 1024 || tpc > RG_THREADS || n_rt > RG_THREADS) return cudaErrorNotSupported;
    a.tiles_per_cta = tpc;
    a.sig_log2e = sigmoid_log2e(a.fa); a.sig_clip = sigmoid_clip(a.fa);
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(routed_gateup_kernel<QT, FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n_tiles + tpc - 1) / tpc)); cfg.blockDim = dim3(RG_THREADS);
    cfg.dynamicSmemBytes = (size_t)L.total; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = a.pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, routed_gateup_kernel<QT, FAST>, a);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

// cudaErrorNotSupported: shape or type outside what the fused launch carries (the caller runs the routing kernel
// and the streamed gate/up kernel instead).
cudaError_t launch_routed_gateup(int qtype, const RoutedGateUpArgs &a, cudaStream_t s) {
    if (a.d <= 0 || a.d % 256 || a.d > 4096 || a.n_experts <= 0 || a.n_experts > 1024 || a.k <= 0 || a.k > a.n_experts ||
        a.k > 64 || a.e_ffn <= 0) return cudaErrorInvalidValue;
    if (qtype != QT_Q4K) return cudaErrorNotSupported;
    return a.fast ? launch_t<QT_Q4K, true>(a, s) : launch_t<QT_Q4K, false>(a, s);
}

}  // namespace iie
