// Grouped expert products for small batches (2 .. ~190 rows): every touched expert tile is streamed ONCE.
//
// The reference's batched entries (north-mini-code/tools/nmc_qk_cuda.cu:2184-2346 matmul_multi_tok and the host
// loop around it) stream a whole expert per (token, expert) pair.  With a few rows per expert the step is still
// bound by the weight bytes, so this kernel keeps the single-token streaming scheme -- a CTA asks the copy engine
// for a run of 16-row tiles up front (cp.async.bulk, one single-use mbarrier per tile) -- and applies each tile,
// once it has landed, to ALL rows routed to its expert: work items are (tile, row) pairs dealt to the warps, a
// warp walks the whole K of its item, so nothing is reduced across warps; the eight digit columns of the 16
// output rows go through a per-warp shared-memory patch to the lanes that run the epilogue (integer SiLU * up
// and digit planes for gate/up, gate-weighted atomic combine for down, plain store for a linear product).
// Experts without rows are skipped before any byte is requested.  Arithmetic and envelopes are those of stream.cu.
#include <algorithm>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"

namespace iie {

namespace {

constexpr int BT_WARPS = 8;                 // two CTAs per SM: one multiplies while the other's tiles stream in
constexpr int BT_SMEM = 108 * 1024;
constexpr unsigned BT_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t bt_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool bt_wait(uint64_t *bar) {
    for (unsigned it = 0; it < BT_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bt_u32(bar)) : "memory");
        if (ok) return true;
    }
    return false;
}

// dense items pay when ceil(rows / 8) * digits walks (each a little dearer than a digit-column walk) undercut one walk per row
__device__ __forceinline__ bool bt_dense(int rows, int digits) { return ((rows + 7) / 8) * digits * 23 < rows * 20; }

template <int QT, int MODE, bool FAST>
__global__ void __launch_bounds__(BT_WARPS * 32, 2) batch_kernel(const BatchArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int nb = (int)a.n_blocks, tile_bytes = 2 * nb * HTB, tpc = a.tiles_per_cta;
    const long long K = a.n_blocks * 256;
    uint8_t *wbuf = smem;
    unsigned long long *patch = reinterpret_cast<unsigned long long *>(smem + (size_t)tpc * tile_bytes);     // [warp][16][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(patch + BT_WARPS * 128);
    int *t_off = reinterpret_cast<int *>(bars + tpc);                 // tile -> first work item; t_off[tpc] = item count
    __shared__ int s_timeout;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int n_ht = (int)((a.out_f + 7) >> 3);
    const int tpe = a.tiles_per_expert;
    const long long tile0 = (long long)blockIdx.x * tpc;
    const int my_tiles = (int)max(0LL, min((long long)tpc, (long long)a.n_groups * tpe - tile0));

    for (int i = tid; i < tpc; i += blockDim.x) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bt_u32(&bars[i])));
    // Digits in use by the activations (8 when unknown).  An expert with enough rows takes "dense" items: eight rows are the
    // eight MMA columns and the item walks K once per digit, so the weight codes are unpacked ceil(rows / 8) * digits times
    // instead of once per row.  bt_dense() decides per expert (the same in every thread).
    const int nl_x = a.x_nl ? max(1, min(8, *a.x_nl)) : 8;
    if (tid == 0) {
        s_timeout = 0;
        int run = 0;
        for (int i = 0; i < my_tiles; i++) {
            const int e = (int)((tile0 + i) / tpe);
            t_off[i] = run;
            const int rows = a.grp_off[e + 1] - a.grp_off[e];
            run += bt_dense(rows, nl_x) ? (rows + 7) / 8 : rows;
        }
        for (int i = my_tiles; i <= tpc; i++) t_off[i] = run;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // one lane per tile requests it, unless its expert has no rows
    if (tid < my_tiles && t_off[tid + 1] > t_off[tid]) {
        const long long tau = tile0 + tid;
        const int e = (int)(tau / tpe), p = (int)(tau - (long long)e * tpe);
        uint8_t *dst = wbuf + (size_t)tid * tile_bytes;
        if (MODE == MODE_GATEUP) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bt_u32(&bars[tid])), "r"((uint32_t)tile_bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(bt_u32(dst)), "l"(a.wa[e] + (size_t)p * nb * HTB), "r"((uint32_t)(nb * HTB)), "r"(bt_u32(&bars[tid])) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(bt_u32(dst + nb * HTB)), "l"(a.wb[e] + (size_t)p * nb * HTB), "r"((uint32_t)(nb * HTB)), "r"(bt_u32(&bars[tid])) : "memory");
        } else {
            const uint32_t bytes = (uint32_t)(((2 * p + 1 < n_ht) ? 2 : 1) * nb * HTB);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bt_u32(&bars[tid])), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(bt_u32(dst)), "l"(a.wa[e] + (size_t)(2 * p) * nb * HTB), "r"(bytes), "r"(bt_u32(&bars[tid])) : "memory");
        }
    }
    const bool half = a.x_nl ? (*a.x_nl <= 4) : false;
    const int n_items = t_off[tpc];
    unsigned long long *mine = patch + warp * 128;
    int ti = 0, nl = 0;
    for (int it = warp; it < n_items; it += BT_WARPS) {
        while (it >= t_off[ti + 1]) ti++;                              // items are ordered by tile
        const long long tau = tile0 + ti;
        const int e = (int)(tau / tpe), p = (int)(tau - (long long)e * tpe);
        const int rows_e = a.grp_off[e + 1] - a.grp_off[e];
        if (bt_dense(rows_e, nl_x)) {
            // ---- dense item: rows pair0 .. pair0 + 7 of this expert are the MMA columns; one walk of K per digit ----------------
            const int pair0 = a.grp_off[e] + 8 * (it - t_off[ti]), last = a.grp_off[e] + rows_e;
            const int pcol = min(pair0 + g, last - 1);                  // a column past the expert's rows repeats the last row (result unused)
            const long long xr = a.xidx ? a.xidx[pcol] : pcol;
            if (!bt_wait(&bars[ti])) { s_timeout = 1; continue; }
            const uint8_t *ua0 = wbuf + (size_t)ti * tile_bytes;
            i128 tot[4] = {0, 0, 0, 0};
            for (int l = 0; l < nl_x; l++) {
                const int8_t *xc = a.xl + (xr * 8 + l) * K;
                int64_t acc[4] = {0, 0, 0, 0};
                for (int b = 0; b < nb; b++) {
                    uint32_t bf[16];
                    load_bfrag<QT, true>(xc + (long long)b * 256, t, bf);
                    const uint8_t *ua = ua0 + (size_t)b * HTB;
                    const uint8_t *ub = (MODE == MODE_GATEUP || 2 * p + 1 < n_ht) ? ua + (size_t)nb * HTB : ua;
                    run_item<QT, FAST>(ua, ub, lane, a.fw, bf, false, acc);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) tot[i] += (i128)acc[i] << (8 * l);
            }
            int64_t y[4];
#pragma unroll
            for (int i = 0; i < 4; i++) y[i] = (int64_t)(tot[i] >> a.fw);
#pragma unroll
            for (int c = 0; c < 2; c++) {                               // this lane's two columns: rows pair0 + 2t, pair0 + 2t + 1
                const int pair = pair0 + 2 * t + c;
                if (pair >= last) continue;
                if (MODE == MODE_GATEUP) {
                    const long long row = (long long)p * 8 + g;         // MMA rows 0..7 gate, 8..15 up of the same output index
                    if (row < a.out_f) {
                        const int64_t yg = y[c], yu = y[2 + c];
                        const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
                        const int64_t gu = mul_shift(sg, yu, a.fa);
                        if (a.out) a.out[(long long)pair * a.out_f + row] = gu;
                        bool ok;
                        const uint64_t dg = balanced_digits8(gu, ok);
                        if (!ok) atomicOr(a.flags, 1);
                        nl = max(nl, digits_used(dg));
#pragma unroll
                        for (int l = 0; l < 8; l++) a.out_limbs[((long long)pair * 8 + l) * a.out_f + row] = (int8_t)(dg >> (8 * l));
                    }
                } else {
#pragma unroll
                    for (int hrow = 0; hrow < 2; hrow++) {
                        const long long row = (long long)p * 16 + g + 8 * hrow;
                        if (row >= a.out_f || (hrow && 2 * p + 1 >= n_ht)) continue;
                        const int64_t yv = y[2 * hrow + c];
                        if (MODE == MODE_LINEAR) a.out[(long long)pair * a.out_f + row] = yv;
                        else {
                            const long long tok = a.pair_tok ? a.pair_tok[pair] : pair;
                            atomicAdd(reinterpret_cast<unsigned long long *>(a.out + tok * a.out_f + row),
                                      (unsigned long long)mul_shift(yv, a.gates[pair], a.fa));
                        }
                    }
                }
            }
            continue;
        }
        const int pair = a.grp_off[e] + (it - t_off[ti]);
        const long long xrow = a.xidx ? a.xidx[pair] : pair;
        const int8_t *xcol = a.xl + (xrow * 8 + col_limb(g)) * K;
        if (!bt_wait(&bars[ti])) { s_timeout = 1; continue; }
        const uint8_t *ua0 = wbuf + (size_t)ti * tile_bytes;
        int64_t acc[4] = {0, 0, 0, 0};
        for (int b = 0; b < nb; b++) {
            uint32_t bf[16];
            load_bfrag<QT, true>(xcol + (long long)b * 256, t, bf);
            const uint8_t *ua = ua0 + (size_t)b * HTB;
            const uint8_t *ub = (MODE == MODE_GATEUP || 2 * p + 1 < n_ht) ? ua + (size_t)nb * HTB : ua;
            run_item<QT, FAST>(ua, ub, lane, a.fw, bf, half, acc);
        }
        __syncwarp();
        mine[g * 8 + 2 * t] = (unsigned long long)acc[0]; mine[g * 8 + 2 * t + 1] = half ? 0ULL : (unsigned long long)acc[1];
        mine[(g + 8) * 8 + 2 * t] = (unsigned long long)acc[2]; mine[(g + 8) * 8 + 2 * t + 1] = half ? 0ULL : (unsigned long long)acc[3];
        __syncwarp();
        if (MODE == MODE_GATEUP) {
            if (lane < 8) {                                             // rows 0..7 gate, 8..15 up of the same output index
                const long long row = (long long)p * 8 + lane;
                if (row < a.out_f) {
                    const int64_t yg = recombine_cols(mine + lane * 8, a.fw), yu = recombine_cols(mine + (lane + 8) * 8, a.fw);
                    const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
                    const int64_t gu = mul_shift(sg, yu, a.fa);
                    if (a.out) a.out[(long long)pair * a.out_f + row] = gu;
                    bool ok;
                    const uint64_t dg = balanced_digits8(gu, ok);
                    if (!ok) atomicOr(a.flags, 1);
                    nl = max(nl, digits_used(dg));
#pragma unroll
                    for (int l = 0; l < 8; l++) a.out_limbs[((long long)pair * 8 + l) * a.out_f + row] = (int8_t)(dg >> (8 * l));
                }
            }
        } else if (lane < 16) {
            const long long row = (long long)p * 16 + lane;
            if (row < a.out_f && (lane < 8 || 2 * p + 1 < n_ht)) {
                const int64_t y = recombine_cols(mine + lane * 8, a.fw);
                if (MODE == MODE_LINEAR) a.out[(long long)pair * a.out_f + row] = y;
                else {
                    const long long tok = a.pair_tok ? a.pair_tok[pair] : pair;
                    atomicAdd(reinterpret_cast<unsigned long long *>(a.out + tok * a.out_f + row),
                              (unsigned long long)mul_shift(y, a.gates[pair], a.fa));
                }
            }
        }
    }
    if (MODE == MODE_GATEUP && a.out_nl) {
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
        nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
        if (lane == 0 && nl > 0) atomicMax(a.out_nl, nl);
    }
    __syncthreads();
    // tiles whose copy was requested must have landed before the CTA may exit (all of them had items, so all
    // were waited for unless a wait timed out)
    if (s_timeout && tid == 0) atomicOr(a.flags, 8);
}

template <int QT, int MODE, bool FAST>
cudaError_t launch_t(const BatchArgs &a_in, cudaStream_t s) {
    BatchArgs a = a_in;
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const long long n_ht = (a.out_f + 7) >> 3;
    a.tiles_per_expert = (int)(MODE == MODE_GATEUP ? n_ht : (n_ht + 1) / 2);
    const size_t tile_bytes = (size_t)2 * a.n_blocks * HTB;
    const size_t fixed = (size_t)BT_WARPS * 1024 + 64;
    int tpc = (int)((BT_SMEM - fixed) / (tile_bytes + 16));
    if (tpc < 1) return cudaErrorNotSupported;
    const long long n_tiles = (long long)a.n_groups * a.tiles_per_expert;
    tpc = (int)std::min<long long>(tpc, std::max<long long>(1, (n_tiles + 295) / 296));
    tpc = std::min(tpc, BT_WARPS * 32);
    a.tiles_per_cta = tpc;
    a.sig_log2e = sigmoid_log2e(a.fa); a.sig_clip = sigmoid_clip(a.fa);
    const size_t smem = (size_t)tpc * tile_bytes + (size_t)BT_WARPS * 1024 + (size_t)tpc * 8 + (size_t)(tpc + 1) * 4 + 16;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(batch_kernel<QT, MODE, FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, BT_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    batch_kernel<QT, MODE, FAST><<<(unsigned)((n_tiles + tpc - 1) / tpc), BT_WARPS * 32, smem, s>>>(a);
    note_launch();
    return cudaGetLastError();
}

template <int QT, int MODE>
cudaError_t launch_f(const BatchArgs &a, cudaStream_t s) {
    return a.fast ? launch_t<QT, MODE, true>(a, s) : launch_t<QT, MODE, false>(a, s);
}

}  // namespace

cudaError_t launch_batch(int qtype, int mode, const BatchArgs &a, cudaStream_t s) {
    if (a.n_groups <= 0 || a.out_f <= 0 || a.n_blocks <= 0 || !a.grp_off) return cudaErrorInvalidValue;
    if (qtype == QT_Q4K) {
        if (mode == MODE_LINEAR) return launch_f<QT_Q4K, MODE_LINEAR>(a, s);
        if (mode == MODE_GATEUP) return launch_f<QT_Q4K, MODE_GATEUP>(a, s);
        return launch_f<QT_Q4K, MODE_DOWN>(a, s);
    }
    if (qtype == QT_Q6K) {
        if (mode == MODE_LINEAR) return launch_f<QT_Q6K, MODE_LINEAR>(a, s);
        if (mode == MODE_GATEUP) return launch_f<QT_Q6K, MODE_GATEUP>(a, s);
        return launch_f<QT_Q6K, MODE_DOWN>(a, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace iie
