// Single-token expert stage in ONE launch: gate/up product + integer SiLU * up, then the down product with the
// gate-weighted combine, one thread-block cluster per selected expert.
//
// Replaces the two streamed launches (and, in the reference, north-mini-code/tools/nmc_qk_cuda.cu:1816-1866
// qk_moe_ffn with its six launches) for the decode step.  The dependency "down needs every gate*up value of
// its expert" is per expert, so it is resolved inside a cluster of 10-16 CTAs with the hardware cluster barrier
// instead of a kernel boundary:
//   * each CTA owns a contiguous run of the expert's gate/up tiles and of its down tiles and asks the copy
//     engine for all of them at once (cp.async.bulk, one single-use mbarrier per tile); when shared memory
//     holds both sets the down weights stream in while the gate/up tiles are being multiplied, otherwise
//     they are requested into the gate/up buffer as soon as its last tile has been read;
//   * gate/up tiles are reduced across the K-split warps in shared memory, the epilogue forms
//     gu = (silu(g) * u) >> fa and its balanced digits, and every CTA pushes its 8-byte digit runs into the
//     shared memory of all CTAs of the cluster (distributed shared memory), together with the digit count it saw;
//   * after the cluster barrier every CTA holds the expert's complete digit planes and multiplies its down
//     tiles; the warp that completes a tile adds floor(y * gate / 2^fa) to the block's output row.
// Clusters never wait for one another, so the launch is correct whether or not all of them are resident.
// Every mbarrier wait is bounded (flag bit 3); the cluster barrier is reached by every thread of every CTA.
#include <cooperative_groups.h>

#include <algorithm>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"

namespace cg = cooperative_groups;

namespace iie {

int g_expert_clusters = -1;            // co-resident clusters of the chosen size (-1: not asked yet)
int g_expert_cluster_size = 0;         // CTAs per cluster the launcher settled on

namespace {

constexpr int EX_WARPS = 16, EX_CLUSTER = 16;          // EX_CLUSTER: largest cluster (sizes the digit-count array)
constexpr unsigned EX_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t ex_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ex_bar_init(uint64_t *bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ex_u32(bar))); }
__device__ __forceinline__ void ex_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ex_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ex_wait(uint64_t *bar) {
    for (unsigned it = 0; it < EX_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(ex_u32(bar)) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void ex_bulk(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ex_u32(dst)), "l"(src), "r"(bytes), "r"(ex_u32(bar)) : "memory");
}

struct ExLayout {                       // byte offsets inside dynamic shared memory
    int wg, wd, red_g, red_d, planes, stage, bars_g, bars_d, done_d, nl_arr, total;
};

__host__ __device__ inline ExLayout ex_layout(int gt, int dt, int tb_g, int tb_d, int e_ffn, int down_early) {
    ExLayout L;
    int o = 0;
    L.wg = o;
    if (down_early) { o += gt * tb_g; L.wd = o; o += dt * tb_d; }
    else { L.wd = o; o += gt * tb_g > dt * tb_d ? gt * tb_g : dt * tb_d; }
    o = (o + 127) & ~127;
    L.red_g = o; o += gt * 1024;
    L.red_d = o; o += dt * 1024;
    L.planes = o; o += 8 * e_ffn;
    L.stage = o; o += 8 * gt * 8;
    o = (o + 7) & ~7;
    L.bars_g = o; o += gt * 8;
    L.bars_d = o; o += dt * 8;
    L.done_d = o; o += dt * 4;
    L.nl_arr = o; o += EX_CLUSTER * 4;
    L.total = o;
    return L;
}

template <int GQT, int DQT>
__global__ void __launch_bounds__(EX_WARPS * 32, 1) expert_kernel(const ExpertArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int HTB_G = GQT == QT_Q4K ? HTB_Q4K : HTB_Q6K, HTB_D = DQT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
    const int slot = (int)(blockIdx.x / csize);
    const int nb_g = (int)(a.d_model / 256), nb_d = (int)(a.e_ffn / 256);
    const int tb_g = 2 * nb_g * HTB_G, tb_d = 2 * nb_d * HTB_D;
    const int gt = a.gt, dt = a.dt;
    const ExLayout L = ex_layout(gt, dt, tb_g, tb_d, (int)a.e_ffn, a.down_early);
    uint8_t *wg = smem + L.wg, *wd = smem + L.wd;
    unsigned long long *red_g = reinterpret_cast<unsigned long long *>(smem + L.red_g);
    unsigned long long *red_d = reinterpret_cast<unsigned long long *>(smem + L.red_d);
    int8_t *planes = reinterpret_cast<int8_t *>(smem + L.planes);
    uint8_t *stage = smem + L.stage;
    uint64_t *bars_g = reinterpret_cast<uint64_t *>(smem + L.bars_g), *bars_d = reinterpret_cast<uint64_t *>(smem + L.bars_d);
    int *done_d = reinterpret_cast<int *>(smem + L.done_d), *nl_arr = reinterpret_cast<int *>(smem + L.nl_arr);
    __shared__ int s_timeout, s_nl;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_g = (int)((a.e_ffn + 7) >> 3);                       // gate/up tiles of the expert (8 gate + 8 up rows each)
    const int n_hd = (int)((a.d_model + 7) >> 3), n_d = (n_hd + 1) >> 1;
    const int g0 = rank * gt, my_g = max(0, min(gt, n_g - g0));
    const int d0 = rank * dt, my_d = max(0, min(dt, n_d - d0));

    for (int i = threadIdx.x; i < gt * 128; i += blockDim.x) red_g[i] = 0ULL;
    for (int i = threadIdx.x; i < dt * 128; i += blockDim.x) red_d[i] = 0ULL;
    for (int i = threadIdx.x; i < gt; i += blockDim.x) ex_bar_init(&bars_g[i]);
    for (int i = threadIdx.x; i < dt; i += blockDim.x) { ex_bar_init(&bars_d[i]); done_d[i] = 0; }
    if (threadIdx.x == 0) { s_timeout = 0; s_nl = 0; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");     // "this CTA runs": waited for before the pushes
    // everything above touched only this CTA's shared memory; the selected pointers, the activation digits
    // and the output row come from the routing kernel
    if (a.pdl) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }

    if (threadIdx.x < my_g) {
        const int i = threadIdx.x;
        const uint8_t *pg = a.sel_ptrs[slot], *pu = a.sel_ptrs[a.k + slot];
        ex_expect(&bars_g[i], (uint32_t)tb_g);
        ex_bulk(wg + (size_t)i * tb_g, pg + (size_t)(g0 + i) * nb_g * HTB_G, (uint32_t)(nb_g * HTB_G), &bars_g[i]);
        ex_bulk(wg + (size_t)i * tb_g + nb_g * HTB_G, pu + (size_t)(g0 + i) * nb_g * HTB_G, (uint32_t)(nb_g * HTB_G), &bars_g[i]);
    }
    auto request_down = [&]() {
        if (threadIdx.x >= 32 && threadIdx.x - 32 < my_d) {
            const int i = threadIdx.x - 32;
            const uint8_t *pd = a.sel_ptrs[2 * a.k + slot];
            const int p = d0 + i, units = (2 * p + 1 < n_hd) ? 2 : 1;
            ex_expect(&bars_d[i], (uint32_t)(units * nb_d * HTB_D));
            ex_bulk(wd + (size_t)i * tb_d, pd + (size_t)(2 * p) * nb_d * HTB_D, (uint32_t)(units * nb_d * HTB_D), &bars_d[i]);
        }
    };
    if (a.down_early) request_down();
    const int g = lane >> 2, t = lane & 3;

    // ---- phase 1: gate/up items (tile, block) dealt round-robin to the warps --------------------------------------
    {
        const bool half = *a.h_nl <= 4;
        const long long xoff = (long long)col_limb(g) * a.d_model;
        uint32_t bf[16];
        int bcur = -1;
        const int n_items = my_g * nb_g;
        for (int it = warp; it < n_items; it += EX_WARPS) {
            const int ti = it / nb_g, b = it - ti * nb_g;
            if (b != bcur) { load_bfrag<GQT, true>(a.hl + xoff + (long long)b * 256, t, bf); bcur = b; }
            const uint8_t *ua = wg + (size_t)ti * tb_g + (size_t)b * HTB_G, *ub = ua + (size_t)nb_g * HTB_G;
            if (!ex_wait(&bars_g[ti])) { s_timeout = 1; continue; }
            int64_t acc[4] = {0, 0, 0, 0};
            run_item<GQT, true>(ua, ub, lane, a.fw, bf, half, acc);
            unsigned long long *r = red_g + (size_t)ti * 128;
            atomicAdd(&r[g * 8 + 2 * t], (unsigned long long)acc[0]);
            atomicAdd(&r[(g + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
            if (!half) {
                atomicAdd(&r[g * 8 + 2 * t + 1], (unsigned long long)acc[1]);
                atomicAdd(&r[(g + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
            }
        }
    }
    __syncthreads();
    if (!a.down_early) request_down();                    // the gate/up tiles have been read: their buffer takes the down tiles
    // ---- epilogue 1: gu and its digits for this CTA's 8 * my_g rows, staged as [digit][row] ------------------------
    {
        int nl = 0;
        for (int idx = threadIdx.x; idx < my_g * 8; idx += blockDim.x) {
            const int tq = idx >> 3, r8 = idx & 7;
            const unsigned long long *rr = red_g + (size_t)tq * 128;
            const int64_t yg = recombine_cols(rr + r8 * 8, a.fw), yu = recombine_cols(rr + (r8 + 8) * 8, a.fw);
            const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
            const int64_t gu = mul_shift(sg, yu, a.fa);
            bool ok;
            const uint64_t d = balanced_digits8(gu, ok);
            if (!ok) atomicOr(a.flags, 1);
            nl = max(nl, digits_used(d));
#pragma unroll
            for (int l = 0; l < 8; l++) stage[l * (gt * 8) + idx] = (uint8_t)(d >> (8 * l));
        }
        if (nl > 0) atomicMax(&s_nl, nl);
    }
    __syncthreads();
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");                 // every CTA of the cluster is running
    // ---- push this CTA's digit runs (8 bytes per tile and digit) and its digit count to all CTAs -------------------
    {
        const int per_peer = 8 * my_g;
        for (int idx = threadIdx.x; idx < csize * per_peer; idx += blockDim.x) {
            const int peer = idx / per_peer, rem = idx - peer * per_peer, l = rem / my_g, tq = rem - l * my_g;
            const unsigned long long v = *reinterpret_cast<const unsigned long long *>(stage + l * (gt * 8) + tq * 8);
            int8_t *dst = cluster.map_shared_rank(planes, peer) + (long long)l * a.e_ffn + (long long)(g0 + tq) * 8;
            *reinterpret_cast<unsigned long long *>(dst) = v;
        }
        if (threadIdx.x < csize) cluster.map_shared_rank(nl_arr, threadIdx.x)[rank] = s_nl;
    }
    cluster.sync();                                                              // release the pushes / acquire the peers'

    // ---- phase 2: down items; the warp that completes a tile adds it to the output row ----------------------------
    {
        int nl = 1;
        for (int i = 0; i < csize; i++) nl = max(nl, nl_arr[i]);
        const bool half = nl <= 4;
        const int64_t gate = a.gates[slot];
        const int8_t *xcol = planes + (long long)col_limb(g) * a.e_ffn;
        uint32_t bf[16];
        int bcur = -1;
        const int n_items = my_d * nb_d;
        for (int it = warp; it < n_items; it += EX_WARPS) {
            const int ti = it / nb_d, b = it - ti * nb_d;
            if (b != bcur) { load_bfrag<DQT, false>(xcol + (long long)b * 256, t, bf); bcur = b; }
            const int p = d0 + ti;
            const uint8_t *ua = wd + (size_t)ti * tb_d + (size_t)b * HTB_D;
            const uint8_t *ub = (2 * p + 1 < n_hd) ? ua + (size_t)nb_d * HTB_D : ua;
            if (!ex_wait(&bars_d[ti])) { s_timeout = 1; continue; }
            int64_t acc[4] = {0, 0, 0, 0};
            run_item<DQT, true>(ua, ub, lane, a.fw, bf, half, acc);
            unsigned long long *r = red_d + (size_t)ti * 128;
            atomicAdd(&r[g * 8 + 2 * t], (unsigned long long)acc[0]);
            atomicAdd(&r[(g + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
            if (!half) {
                atomicAdd(&r[g * 8 + 2 * t + 1], (unsigned long long)acc[1]);
                atomicAdd(&r[(g + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
            }
            __threadfence_block();
            int prior = 0;
            if (lane == 0) prior = atomicAdd(&done_d[ti], 1);
            prior = __shfl_sync(0xffffffffu, prior, 0);
            if (prior != nb_d - 1) continue;
            __threadfence_block();
            const volatile unsigned long long *rv = r;
            if (lane < 16) {
                const long long row = (long long)p * 16 + lane;
                if (row < a.d_model && (lane < 8 || 2 * p + 1 < n_hd)) {
                    unsigned long long cc[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) cc[c] = rv[lane * 8 + c];
                    const int64_t y = recombine_cols(cc, a.fw);
                    atomicAdd(reinterpret_cast<unsigned long long *>(a.out + row), (unsigned long long)mul_shift(y, gate, a.fa));
                }
            }
        }
    }
    __syncthreads();
    if (s_timeout && threadIdx.x == 0) atomicOr(a.flags, 8);
}

template <int GQT, int DQT>
cudaError_t launch_t(const ExpertArgs &a_in, cudaStream_t s) {
    ExpertArgs a = a_in;
    constexpr int HTB_G = GQT == QT_Q4K ? HTB_Q4K : HTB_Q6K, HTB_D = DQT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int nb_g = (int)(a.d_model / 256), nb_d = (int)(a.e_ffn / 256);
    const int n_g = (int)((a.e_ffn + 7) >> 3), n_d = (int)((((a.d_model + 7) >> 3) + 1) >> 1);
    constexpr int MAX_SMEM = 225 * 1024;
    static int clusters_for[EX_CLUSTER + 1];                  // 0 not asked, -1 unusable, else co-resident clusters
    static bool attrs_set = false;
    if (!attrs_set) {
        if (cudaFuncSetAttribute(expert_kernel<GQT, DQT>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(expert_kernel<GQT, DQT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
            cudaGetLastError(); return cudaErrorNotSupported;
        }
        attrs_set = true;
    }
    // the largest cluster whose clusters can all be resident at once; else the one keeping most SMs busy
    int best = 0, best_score = 0, best_early = 0;
    for (int cs = EX_CLUSTER; cs >= 10; cs -= 2) {
        const int gt = (n_g + cs - 1) / cs, dt = (n_d + cs - 1) / cs;
        if (gt > 32 || dt > 256) continue;
        int early = 1;
        ExLayout L = ex_layout(gt, dt, 2 * nb_g * HTB_G, 2 * nb_d * HTB_D, (int)a.e_ffn, 1);
        if (L.total > MAX_SMEM) { early = 0; L = ex_layout(gt, dt, 2 * nb_g * HTB_G, 2 * nb_d * HTB_D, (int)a.e_ffn, 0); }
        if (L.total > MAX_SMEM) continue;
        if (clusters_for[cs] == 0) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3((unsigned)(a.k * cs)); probe.blockDim = dim3(EX_WARPS * 32); probe.dynamicSmemBytes = (size_t)L.total;
            cudaLaunchAttribute pa[1];
            pa[0].id = cudaLaunchAttributeClusterDimension;
            pa[0].val.clusterDim.x = (unsigned)cs; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
            probe.attrs = pa; probe.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, expert_kernel<GQT, DQT>, &probe) != cudaSuccess || n < 1) { cudaGetLastError(); n = -1; }
            clusters_for[cs] = n;
        }
        if (clusters_for[cs] < 1) continue;
        const int score = (clusters_for[cs] >= a.k ? 1000 : 0) + std::min(clusters_for[cs], a.k) * cs;
        if (score > best_score) { best_score = score; best = cs; best_early = early; }
        if (clusters_for[cs] >= a.k) break;
    }
    if (best == 0 || clusters_for[best] < a.k) return cudaErrorNotSupported;   // a second wave would cost more than two launches
    g_expert_clusters = clusters_for[best]; g_expert_cluster_size = best;
    a.gt = (n_g + best - 1) / best; a.dt = (n_d + best - 1) / best; a.down_early = best_early;
    const ExLayout L = ex_layout(a.gt, a.dt, 2 * nb_g * HTB_G, 2 * nb_d * HTB_D, (int)a.e_ffn, best_early);
    a.sig_log2e = sigmoid_log2e(a.fa); a.sig_clip = sigmoid_clip(a.fa);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.k * best)); cfg.blockDim = dim3(EX_WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)L.total; cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)best; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = a.pdl ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, expert_kernel<GQT, DQT>, a);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

// cudaErrorNotSupported: no instantiation for this pair of types / shape, or 16-CTA clusters are not available
// (the caller then uses the two streamed launches).
cudaError_t launch_expert(int gate_q, int down_q, const ExpertArgs &a, cudaStream_t s) {
    if (a.k <= 0 || a.d_model <= 0 || a.e_ffn <= 0 || a.d_model % 256 || a.e_ffn % 256) return cudaErrorInvalidValue;
    if (gate_q == QT_Q4K && down_q == QT_Q6K) return launch_t<QT_Q4K, QT_Q6K>(a, s);
    if (gate_q == QT_Q4K && down_q == QT_Q4K) return launch_t<QT_Q4K, QT_Q4K>(a, s);
    return cudaErrorNotSupported;
}

}  // namespace iie
