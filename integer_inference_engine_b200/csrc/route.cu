// Fused single-token routing: RMSNorm -> limb planes -> quantised router product -> top-k with
// lowest-index tie-break -> sigmoid gates, in one launch.
//
// Replaces the reference's five-launch sequence rmsnorm_fast_u64_k / rmsnorm_exact_k /
// router_fast_i64_k / router_i64_k / topk_lowidx_k (north-mini-code/tools/nmc_qk_cuda.cu:434-657,
// host entry :1116-1173) for the configuration in which the router itself is a Q4_K / Q6_K tensor.
// Arithmetic: north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72 (RMSNorm), cohere2.py:162-180
// (routing).  Every CTA recomputes the (tiny) normalisation so that no grid-wide barrier is needed
// before the router rows; the CTA that finishes last performs the top-k.
#include <cooperative_groups.h>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"
#include "norm.cuh"

namespace cg = cooperative_groups;

namespace iie {

namespace {

constexpr int RT_THREADS = 256;
constexpr int RT_MAX_D = 4096;            // elements of one row staged per CTA (tile + planes + x + gain fit shared memory)
constexpr int RT_PAD = 32;                // plane padding (bytes): keeps the 8 limb planes on different banks

__device__ __forceinline__ uint32_t rt_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// rank of element e among n logits: how many beat it (greater, or equal with a lower index)
__device__ __forceinline__ int rank_part(const int64_t *lg, int e, int64_t v, int j0, int j1) {
    int rank = 0;
    for (int j = j0; j < j1; j++) {
        const int64_t w = lg[j];
        rank += (w > v) || (w == v && j < e);
    }
    return rank;
}

template <int QT, bool CLUSTER>
__global__ void __launch_bounds__(RT_THREADS) route_kernel(const RouteArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int d = a.d, stride = d + RT_PAD, nb = d / 256;
    uint8_t *wtile = smem;                                                     // this CTA's router tile: 2 units x nb blocks
    int8_t *planes = reinterpret_cast<int8_t *>(smem + (size_t)2 * nb * HTB);  // [8][stride]
    int64_t *xs = reinterpret_cast<int64_t *>(planes + (size_t)8 * stride);    // [d] staged input row
    int64_t *gs = xs + d;                                                      // [d] staged gain
    __shared__ unsigned long long s_lo[RT_THREADS / 32], s_hi[RT_THREADS / 32], s_max[RT_THREADS / 32], s_gmax[RT_THREADS / 32];
    __shared__ unsigned long long s_rms, s_inv, s_gm;
    __shared__ int s_bad, s_nl, s_last, s_timeout;
    __shared__ unsigned long long red[16][8];
    __shared__ int64_t s_logits[1024];
    __shared__ __align__(8) uint64_t s_bar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- before the dependency wait: everything that reads only immutable data ---------------------------
    const long long n_ht = ((long long)a.n_experts + 7) >> 3;
    const long long htA = 2LL * blockIdx.x, htB = htA + 1 < n_ht ? htA + 1 : htA;
    if (tid == 0) {
        s_bad = 0; s_nl = 1; s_last = 0; s_timeout = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rt_smem_u32(&s_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint32_t bytes = (uint32_t)((htB != htA ? 2 : 1) * nb * HTB);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rt_smem_u32(&s_bar)), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(rt_smem_u32(wtile)), "l"(a.router + (size_t)htA * nb * HTB), "r"(bytes), "r"(rt_smem_u32(&s_bar)) : "memory");
    }
    for (int i = tid; i < 128; i += RT_THREADS) (&red[0][0])[i] = 0ULL;
    if (a.tabs && blockIdx.x == 0)                       // warm the layer's pointer tables in L2 for the tail of this kernel
        for (int i = tid * 16; i < 3 * a.n_experts; i += RT_THREADS * 16)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.tabs + i));
    unsigned long long gmx = 0;
    if (a.gain)
        for (int i = tid * 2; i < d; i += RT_THREADS * 2) {
            const longlong2 gv = *reinterpret_cast<const longlong2 *>(a.gain + i);
            *reinterpret_cast<longlong2 *>(gs + i) = gv;
            const unsigned long long g0 = uabs64(gv.x), g1 = uabs64(gv.y);
            gmx = g0 > gmx ? g0 : gmx; gmx = g1 > gmx ? g1 : gmx;
        }
    if (a.pdl) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;"); }

    // ---- stage x, sum of squares and magnitudes -------------------------------------------------------
    {
        u128 ssq = 0; unsigned long long mx = 0;
        for (int i = tid * 2; i < d; i += RT_THREADS * 2) {
            const longlong2 xv = *reinterpret_cast<const longlong2 *>(a.x + i);
            *reinterpret_cast<longlong2 *>(xs + i) = xv;
            const unsigned long long v0 = uabs64(xv.x), v1 = uabs64(xv.y);
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
                for (int i = 0; i < RT_THREADS / 32; i++) {
                    total += ((u128)s_hi[i] << 64) | s_lo[i];
                    m = s_max[i] > m ? s_max[i] : m; gm = s_gmax[i] > gm ? s_gmax[i] : gm;
                }
                if (m > (1ULL << 57)) s_bad = 1;                 // keeps the 128-bit sum of squares exact
                u128 mean;
                if ((d & (d - 1)) == 0) mean = total >> (31 - __clz(d));        // widths are powers of two in practice
                else if ((total >> 64) == 0) mean = (u128)((unsigned long long)total / (unsigned long long)d);
                else mean = total / (u128)(unsigned long long)d;
                const u128 rms = isqrt128(mean + a.eps);
                if (rms == 0 || rms > (u128)0xFFFFFFFFFFFFFFFFULL) s_bad = 1;
                s_rms = (unsigned long long)rms; s_gm = gm;
                s_inv = rms != 0 ? 0xFFFFFFFFFFFFFFFFULL / (unsigned long long)rms : 0;
            }
        }
    }
    __syncthreads();
    if (s_bad) { if (tid == 0 && blockIdx.x == 0) atomicOr(a.flags, 2); return; }   // uniform over the grid

    // ---- normalise, apply the gain, split into limb planes (four consecutive elements per step) ------------
    const unsigned long long rms = s_rms, inv = s_inv, gm = s_gm;
    bool bad = false, over = false;
    int nl = 1;
    for (int i = tid * 4; i < d; i += RT_THREADS * 4) {
        uint32_t pw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int64_t yv[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int64_t xv = xs[i + e];
            int64_t y = xv;
            if (a.gain) {
                if (uabs64(xv) < (1ULL << (62 - a.fa)) && rms < (1ULL << 62)) y = floor_div_recip(xv * ((long long)1 << a.fa), rms, inv);
                else {
                    const i128 num = (i128)xv * ((i128)1 << a.fa);
                    i128 q = num / (i128)rms;
                    if (num < 0 && q * (i128)rms != num) q -= 1;
                    if (q > (i128)INT64_MAX || q < (i128)INT64_MIN) { bad = true; q = 0; }
                    y = (int64_t)q;
                }
                if ((u128)uabs64(y) * gm > (u128)INT64_MAX) bad = true;      // the oracle refuses such a gain product
                y = mul_shift(y, gs[i + e], a.fa);
            }
            yv[e] = y;
            bool ok;
            const uint64_t dg = balanced_digits8(y, ok);
            over |= !ok;
            nl = max(nl, digits_used(dg));
#pragma unroll
            for (int l = 0; l < 8; l++) pw[l] |= (uint32_t)((dg >> (8 * l)) & 0xFF) << (8 * e);
        }
#pragma unroll
        for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * stride + i) = pw[l];
        if (blockIdx.x == 0) {
#pragma unroll
            for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(a.hl + (long long)l * d + i) = pw[l];
            if (a.h_out) { for (int e = 0; e < 4; e++) a.h_out[i + e] = yv[e]; }
            if (a.init_out && a.init_mode)
                for (int e = 0; e < 4; e++) a.init_out[i + e] = a.init_mode == 2 ? xs[i + e] : 0;
        }
    }
    if (bad) atomicOr(a.flags, 2);
    if (over) atomicOr(a.flags, 1);
    nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 16)); nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 8));
    nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 4));  nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 2));
    nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, 1));
    if (lane == 0) atomicMax(&s_nl, nl);
    __syncthreads();
    if (blockIdx.x == 0 && tid == 0) { *a.h_nl = s_nl; if (a.gu_nl) *a.gu_nl = 0; }
    const bool half = s_nl <= 4;

    // ---- router rows of this CTA: one 16-row tile, K split over the warps ------------------------------
    const int g = lane >> 2, t = lane & 3;
    int64_t acc[4] = {0, 0, 0, 0};
    bool arrived = false;
    for (unsigned it = 0; it < (1u << 22) && !arrived; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(rt_smem_u32(&s_bar)) : "memory");
        arrived = ok != 0;
    }
    if (!arrived) s_timeout = 1;
    else
        for (int b = warp; b < nb; b += RT_THREADS / 32) {
            uint32_t bf[16];
            load_bfrag<QT, false>(planes + col_limb(g) * stride + b * 256, t, bf);
            const uint8_t *ua = wtile + (size_t)b * HTB, *ub = htB != htA ? ua + (size_t)nb * HTB : ua;
            run_item<QT, false>(ua, ub, lane, a.fw, bf, half, acc);
        }
    atomicAdd(&red[g][2 * t], (unsigned long long)acc[0]);
    atomicAdd(&red[g + 8][2 * t], (unsigned long long)acc[2]);
    if (!half) {
        atomicAdd(&red[g][2 * t + 1], (unsigned long long)acc[1]);
        atomicAdd(&red[g + 8][2 * t + 1], (unsigned long long)acc[3]);
    }
    __syncthreads();
    if (s_timeout && tid == 0) atomicOr(a.flags, 8);

    const int64_t log2e = sigmoid_log2e(a.fa), clip = sigmoid_clip(a.fa);
    const int n = a.n_experts;
    if (CLUSTER) {
        // ---- every CTA of the cluster receives all logits through distributed shared memory, then ranks
        //      its own 16 rows: sixteen threads per row each compare against a slice of the logits
        cg::cluster_group cluster = cg::this_cluster();
        const unsigned nranks = cluster.num_blocks();
        if (tid < 16) {
            const long long row = (tid < 8 ? htA : htB) * 8 + (tid & 7);
            if (row < n && (tid < 8 || htB != htA)) {
                const int64_t v = recombine_cols(red[tid], a.fw);
                for (unsigned r = 0; r < nranks; r++) cluster.map_shared_rank(s_logits, r)[row] = v;
            }
        }
        cluster.sync();
        const int el = tid >> 4, part = tid & 15;
        const long long row = (el < 8 ? htA : htB) * 8 + (el & 7);
        const bool live = row < n && (el < 8 || htB != htA);
        const int64_t v = live ? s_logits[row] : 0;
        const int per = (n + 15) >> 4, j0 = min(n, part * per), j1 = min(n, j0 + per);
        int rank = live ? rank_part(s_logits, (int)row, v, j0, j1) : 0;
        rank += __shfl_xor_sync(0xffffffffu, rank, 8); rank += __shfl_xor_sync(0xffffffffu, rank, 4);
        rank += __shfl_xor_sync(0xffffffffu, rank, 2); rank += __shfl_xor_sync(0xffffffffu, rank, 1);
        if (live && part == 0 && rank < a.k) {
            a.ids[rank] = (int)row; a.gates[rank] = sigmoid_fixed_c(v, a.fa, log2e, clip);
            if (a.sel_ptrs)
                for (int m = 0; m < 3; m++) a.sel_ptrs[m * a.k + rank] = a.tabs[(size_t)m * n + row];
        }
    } else {
        // ---- no cluster: the CTA that finishes last ranks everything ---------------------------------
        if (tid < 16) {
            const long long row = (tid < 8 ? htA : htB) * 8 + (tid & 7);
            if (row < n && (tid < 8 || htB != htA)) a.logits[row] = recombine_cols(red[tid], a.fw);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned ticket = atomicAdd(a.counter, 1u);
            if (ticket == gridDim.x - 1) { s_last = 1; *a.counter = 0; }
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        for (int i = tid; i < n; i += RT_THREADS) s_logits[i] = *((volatile int64_t *)&a.logits[i]);
        __syncthreads();
        for (int e = tid; e < n; e += RT_THREADS) {
            const int64_t v = s_logits[e];
            const int rank = rank_part(s_logits, e, v, 0, n);
            if (rank < a.k) {
                a.ids[rank] = e; a.gates[rank] = sigmoid_fixed_c(v, a.fa, log2e, clip);
                if (a.sel_ptrs)
                    for (int m = 0; m < 3; m++) a.sel_ptrs[m * a.k + rank] = a.tabs[(size_t)m * n + e];
            }
        }
    }
}

}  // namespace

cudaError_t launch_route(const RouteArgs &a, cudaStream_t s) {
    if (a.d <= 0 || a.d % 256 || a.d > RT_MAX_D || a.n_experts <= 0 || a.n_experts > 1024 || a.k <= 0 ||
        a.k > a.n_experts) return cudaErrorInvalidValue;
    const unsigned grid = (unsigned)((((a.n_experts + 7) >> 3) + 1) / 2);
    const int HTB = a.router_q == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const size_t smem = (size_t)2 * (a.d / 256) * HTB + (size_t)8 * (a.d + RT_PAD) + (size_t)16 * a.d;
    const bool use_cluster = grid <= 8;
    void (*kern)(RouteArgs) = nullptr;
    if (a.router_q == QT_Q4K) kern = use_cluster ? route_kernel<QT_Q4K, true> : route_kernel<QT_Q4K, false>;
    else if (a.router_q == QT_Q6K) kern = use_cluster ? route_kernel<QT_Q6K, true> : route_kernel<QT_Q6K, false>;
    else return cudaErrorInvalidValue;
    static bool configured[2][2] = {{false, false}, {false, false}};
    bool &cfg = configured[a.router_q == QT_Q6K][use_cluster];
    if (!cfg) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
        if (e != cudaSuccess) return e;
        cfg = true;
    }
    cudaLaunchConfig_t cfgl = {};
    cfgl.gridDim = dim3(grid); cfgl.blockDim = dim3(RT_THREADS); cfgl.dynamicSmemBytes = smem; cfgl.stream = s;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (use_cluster) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = grid; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        n_attr = 1;
    }
    if (a.pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfgl.attrs = attr; cfgl.numAttrs = n_attr;
    const cudaError_t e = cudaLaunchKernelEx(&cfgl, kern, a);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace iie
