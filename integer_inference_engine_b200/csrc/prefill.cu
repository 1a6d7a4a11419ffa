// Prefill-regime grouped expert products on the 5th-generation tensor cores (tcgen05, kind::i8).
//
// Replaces the reference's pair-parallel prefill kernels (north-mini-code/tools/nmc_qk_cuda.cu:2184-2201
// matmul_multi_tok / combine_tok and the host loop :2203-2346), which stream one expert's weights once
// per (token, expert) pair, with expert-grouped GEMMs whose weights are dequantised once per tile.
//
// Exactness on an int8 x int8 -> int32 tensor core.  Inside the fast envelope a dequantised weight
// W = d_q*sc*q - dmin_q*m (Q4_K) or d_q*sc*(q-32) (Q6_K) fits NWL balanced base-256 digits and an
// activation fits NL digits, so  sum_k W[n,k] x[m,k] = sum_{a<NWL, b<NL} 256^(a+b) sum_k Wa[n,k] xb[m,k].
// Every digit pair (a,b) is one int8 MMA; pairs with equal a+b share a TMEM accumulator (at most
// min(NWL,NL) pairs x K x 128 x 128 < 2^31 for K <= 8192), the accumulation runs over the FULL K, and the
// epilogue forms sum_s 256^s acc_s in 128 bits and performs the reference's single floor shift.
//
// Tile: 128 weight rows (MMA M, TMEM lanes) x BN (token, expert) pairs (MMA N, TMEM columns) x K in chunks of 64.  The
// weights sit on the wide side because a dequantised weight costs 0.56 bytes of traffic per element and an activation NL
// bytes: the pair side is the one TMEM limits (accumulators x BN <= 512 columns), so it carries the expensive operand.
// Three groups of four warps produce, one shared-memory stage each: one thread asks the copy engine (TMA, 64-byte
// swizzle) for the activation digit planes of the tile's pairs (B operand), and every thread dequantises + digit-splits
// the 64 chunk columns of its weight row into the canonical K-major layout (A operand); then the groups run the epilogue,
// one TMEM lane = one weight row each.  The last warps allocate TMEM and issue the MMAs; tcgen05.commit hands a stage back
// to its group.  Gate and up rows share a tile (lanes 0..63 gate, 64..127 up) and trade halves of their columns through
// shared memory, so the integer SiLU * up product is formed in the epilogue by all 128 threads.
// Activation rows reached through an index (pair -> token) are first gathered into pair order, NL planes per pair, so
// that a tile's rows are consecutive for the copy engine.
// Every wait is bounded; on a time-out the CTA raises flag bit 3, leaves its loops, frees TMEM and exits.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"

namespace iie {

unsigned long long g_prefill_launches[PF_SHAPES];
__device__ long long d_tr[4200];
__device__ int d_tr_block = -1;
__device__ int d_tr_mode = 2;
__device__ int d_pf_exp;
#define TR(i) do { if (trace) d_tr[i] = clock64(); } while (0)

namespace {

constexpr int PF_BM = 128, PF_KC = 64;
constexpr int PF_GROUPS = 3;                              // producer groups of 128 threads; group g fills chunks g, g + 3, ...
constexpr int PF_MAX_STAGES = 6;
constexpr int PF_SMEM_BUDGET = 230 * 1024;                // dynamic shared memory a CTA may ask for, less the alignment slack and the static part
// stages of a tile shape: as many as fit (more stages than groups, so that a group dequantises its next chunk while the
// MMAs of its previous one are still queued)
__host__ __device__ constexpr int pf_stages(int stage_bytes) { return PF_SMEM_BUDGET / stage_bytes < PF_MAX_STAGES ? PF_SMEM_BUDGET / stage_bytes : PF_MAX_STAGES; }
constexpr int PF_ISSUERS = 3;                              // MMA-issuing warps: accumulator s belongs to issuer s % 3
constexpr int PF_THREADS = PF_GROUPS * 128 + PF_ISSUERS * 32;
constexpr unsigned PF_WAIT_LIMIT = 1u << 24;
__device__ __forceinline__ uint32_t pf_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pf_bar_init(uint64_t *b, int n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_u32(b)), "r"(n)); }
__device__ __forceinline__ void pf_bar_arrive(uint64_t *b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pf_u32(b)) : "memory"); }
__device__ __forceinline__ bool pf_bar_wait(uint64_t *b, uint32_t parity, volatile int *abort_flag) {
    for (unsigned it = 0; it < PF_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(pf_u32(b)), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; LBO = distance of
// the two 16-byte K halves of one MMA, SBO = distance of consecutive 8-row groups (bytes, 16-byte units).
__device__ __forceinline__ uint64_t pf_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}

// D[tmem] (+)= A[smem] * B[smem]^T, int8 x int8 -> int32, M = 128, K = 32
__device__ __forceinline__ void pf_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void pf_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pf_u32(bar)) : "memory");
}
__device__ __forceinline__ void pf_tmem_ld8(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

// four int32 weights -> one word per digit plane (byte i of plane l = digit l of weight i)
// (the weights arrive with 0x80808080 already added: byte l of (w + 0x80808080) ^ 0x80808080 is the balanced digit l)
__device__ __forceinline__ void digits4(const uint32_t (&v)[4], uint32_t (&plane)[4]) {
    const uint32_t t0 = __byte_perm(v[0], v[1], 0x5140), t1 = __byte_perm(v[2], v[3], 0x5140);
    const uint32_t t2 = __byte_perm(v[0], v[1], 0x7362), t3 = __byte_perm(v[2], v[3], 0x7362);
    plane[0] = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u; plane[1] = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
    plane[2] = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u; plane[3] = __byte_perm(t2, t3, 0x7632) ^ 0x80808080u;
}

// Dequantise 32 consecutive-k weights of one row into NWL digit planes (eight words each).
// Q4_K: chunk = group G of a block; hsel 0 = low nibbles (first 32 columns), 1 = high nibbles.
struct Q4Raw { uint4 meta; uint2 q[4]; };                 // the 48 bytes of one (row, group) of a repacked Q4_K unit

__device__ __forceinline__ void load_q4k(const uint8_t *unit, int rr, int G, Q4Raw &raw) {
    raw.meta = ldg128(unit + 1024 + rr * 16);
    const uint8_t *qp = unit + (G >> 1) * 512 + rr * 64 + (G & 1) * 8;
#pragma unroll
    for (int t = 0; t < 4; t++) raw.q[t] = ldg64(qp + t * 16);                       // qs[32G + 8t .. +7]
}

template <int NWL>
__device__ __forceinline__ void expand_q4k(const Q4Raw &raw, int G, int hsel, int fw, uint32_t (&pl)[NWL][8]) {
    uint32_t sc0, sc1, mn0, mn1;
    q4k_scales(raw.meta.y, raw.meta.z, raw.meta.w, sc0, sc1, mn0, mn1);
    const int j = 2 * G + hsel;
    const int ws = scale_small(raw.meta.x & 0xFFFF, fw) * (int)(((j < 4 ? sc0 : sc1) >> (8 * (j & 3))) & 0xFF);
    const int wm = scale_small(raw.meta.x >> 16, fw) * (int)(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xFF);
    const uint32_t bias = 0x80808080u - (uint32_t)wm;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const uint32_t words[2] = {(raw.q[t].x >> (4 * hsel)) & 0x0f0f0f0fu, (raw.q[t].y >> (4 * hsel)) & 0x0f0f0f0fu};
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] = (uint32_t)ws * ((words[h2] >> (8 * i)) & 0xFF) + bias;
            uint32_t p4[4];
            digits4(w, p4);
#pragma unroll
            for (int l = 0; l < 4; l++) pl[l][t * 2 + h2] = p4[l];
            if (NWL > 4) pl[NWL - 1][t * 2 + h2] = 0;
        }
    }
}

// Q6_K: chunk cc (0..3) of a block covers half h = cc >> 1 and kq = 2*(cc & 1) + hsel for the two 32-column halves hsel.
// |W| = |d_q sc (q-32)| can need a fifth digit, so the split adds 0x80...80 over 40 bits: byte l of
// (w + 0x8080808080) ^ 0x80..80 is the balanced digit l for |w| <= 127*(256^5-1)/255.  The bias and the -32 ride in the
// addend of the one 32x32->64 multiply-add per weight.  The row's 64 columns are written straight to the five planes of
// the stage (plane stride PLANE): vector (hsel, u) = 16 columns, four words per plane.
template <int PLANE>
__device__ __forceinline__ void dequant64_q6k_store(const uint8_t *unit, int rr, int cc, int fw, uint8_t *wdst) {
    const int h = cc >> 1, hi_nib = cc & 1;
    const int dq = scale_small(__ldg(reinterpret_cast<const unsigned short *>(unit + 1664 + rr * 2)), fw);
    const uint32_t sc4 = __ldg(reinterpret_cast<const uint32_t *>(unit + 1536 + rr * 16 + 8 * h + 4 * hi_nib));   // scales of (hsel, u)
    uint4 lw[4];
    uint2 hb2[4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
        lw[t] = ldg128(unit + h * 512 + (rr * 4 + t) * 16);                             // u0:{first 32, second 32} u1:{..}
        const uint4 hw = ldg128(unit + 1024 + (rr * 4 + t) * 16);                       // [h*2+u]
        hb2[t] = h ? make_uint2(hw.z, hw.w) : make_uint2(hw.x, hw.y);
    }
#pragma unroll
    for (int hsel = 0; hsel < 2; hsel++) {
        const int kq = 2 * hi_nib + hsel;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int ws = dq * (int)(int8_t)(sc4 >> (8 * (2 * hsel + u)));             // |ws| < 2^31 inside the envelope
            const int64_t bias = 0x8080808080LL - 32 * (int64_t)ws;
            uint32_t pl[5][4];
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const uint32_t n = hsel ? (u ? lw[t].w : lw[t].y) : (u ? lw[t].z : lw[t].x);
                const uint32_t hb = u ? hb2[t].y : hb2[t].x;
                const uint32_t q = ((hi_nib ? n >> 4 : n) & 0x0f0f0f0fu) | (((hb >> (2 * kq)) << 4) & 0x30303030u);
                uint32_t vlo[4], vhi[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int64_t uu = (int64_t)ws * (int64_t)(int)((q >> (8 * i)) & 0xFF) + bias;
                    vlo[i] = (uint32_t)uu; vhi[i] = (uint32_t)((uint64_t)uu >> 32);
                }
                const uint32_t t0 = __byte_perm(vlo[0], vlo[1], 0x5140), t1 = __byte_perm(vlo[2], vlo[3], 0x5140);
                const uint32_t t2 = __byte_perm(vlo[0], vlo[1], 0x7362), t3 = __byte_perm(vlo[2], vlo[3], 0x7362);
                pl[0][t] = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u; pl[1][t] = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
                pl[2][t] = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u; pl[3][t] = __byte_perm(t2, t3, 0x7632) ^ 0x80808080u;
                pl[4][t] = __byte_perm(__byte_perm(vhi[0], vhi[1], 0x0040), __byte_perm(vhi[2], vhi[3], 0x0040), 0x5410) ^ 0x80808080u;
            }
#pragma unroll
            for (int l = 0; l < 5; l++)
                *reinterpret_cast<uint4 *>(wdst + hsel * (PLANE / 2) + l * PLANE + u * (PLANE / 4)) = make_uint4(pl[l][0], pl[l][1], pl[l][2], pl[l][3]);
        }
    }
}

// Descriptor of an activation digit plane as the copy engine wrote it: rows of 64 bytes (the whole chunk), 64-byte swizzle,
// eight-row groups 512 bytes apart.  The second K step of a chunk starts 32 bytes into the rows.
__device__ __forceinline__ uint64_t pf_desc_sw64(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ULL << 16) | ((uint64_t)(512 >> 4) << 32) | (1ULL << 46) | (4ULL << 61);
}
__device__ __forceinline__ void pf_expect_tx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pf_u32(b)), "r"(bytes) : "memory");
}
// rows [row, row + BN) of plane `plane`, columns [col, col + 64) of a [rows][planes][K] byte tensor -> shared memory
__device__ __forceinline__ void pf_tma_plane(void *dst, const CUtensorMap *map, int col, int plane, int row, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(pf_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(col), "r"(plane), "r"(row), "r"(pf_u32(bar)) : "memory");
}
__device__ __forceinline__ void pf_group_sync(int group) { asm volatile("bar.sync %0, 128;" ::"r"(1 + group) : "memory"); }

// floor(sum_s r_s 256^s / 2^fw), low 64 bits, for fw <= 32: four accumulators at a time fit int64 (|.| < 2^56), and a
// group's factor 2^(32 g) is a whole multiple of 2^fw from the second group on, so only the first group is floored.
template <int NACC>
__device__ __forceinline__ int64_t pf_recombine(const int (&r)[NACC][8], int j, int fw) {
    uint64_t y = 0;
#pragma unroll
    for (int g = 0; g * 4 < NACC; g++) {
        int64_t v = r[4 * g][j];
#pragma unroll
        for (int t = 1; t < 4; t++)
            if (4 * g + t < NACC) v += (int64_t)r[4 * g + t][j] * (int64_t)(1 << (8 * t));
        if (g == 0) y = (uint64_t)(v >> fw);
        else { const int sh = 32 * g - fw; if (sh < 64) y += (uint64_t)v << sh; }
    }
    return (int64_t)y;
}

// pair -> digit planes in pair order: dst[pair][NL][K] = src[xidx[pair]][0..NL-1][K] (the planes of a row are contiguous).
// Only the pairs the groups own exist (the grid covers the caller's upper bound); `n_live` points at their count.
__global__ void __launch_bounds__(128) gather_planes_kernel(const int8_t *__restrict__ src, const int *__restrict__ xidx, int8_t *__restrict__ dst,
                                                            long long row_bytes, long long src_stride, const int *__restrict__ n_live) {
    const long long pair = blockIdx.x;
    if (pair >= *n_live) return;
    const uint4 *s = reinterpret_cast<const uint4 *>(src + (long long)xidx[pair] * src_stride);
    uint4 *d = reinterpret_cast<uint4 *>(dst + pair * row_bytes);
    for (long long i = threadIdx.x; i < row_bytes / 16; i += 128) d[i] = __ldg(s + i);
}

template <int QT, int MODE, int NL, int NWL, int BN>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const PrefillArgs a, const __grid_constant__ CUtensorMap xmap) {
    constexpr int NACC = NL + NWL - 1;
    static_assert(NACC * BN <= 512 && BN % 16 == 0, "accumulators exceed TMEM");
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    constexpr int W_PLANE = 2 * 2 * (PF_BM / 8) * 128;        // weights: [kstep][khalf][row group][8 rows x 16 B] = 8192
    constexpr int X_PLANE = BN * PF_KC;                        // activations: BN rows of 64 bytes (swizzled by the copy engine)
    constexpr int STAGE_BYTES = NWL * W_PLANE + NL * X_PLANE;
    constexpr int STAGES = pf_stages(STAGE_BYTES);
    static_assert(STAGES >= 3, "a tile shape needs three stages");
    static_assert(X_PLANE % 512 == 0 && STAGE_BYTES % 1024 == 0, "operand tiles must keep the swizzle alignment");
    constexpr int NROW = MODE == MODE_GATEUP ? PF_BM / 2 : PF_BM;   // output rows of one tile
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[PF_MAX_STAGES], empty_bar[PF_MAX_STAGES], accum_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_tile[3];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ex = d_pf_exp; (void)ex;
    const bool tron = (int)blockIdx.x == d_tr_block && MODE == d_tr_mode;
    const bool trace = tron && (tid & 127) == 0;
    if (tid == 0) TR(4002);
    const int nb = (int)a.n_blocks, K = nb * 256, n_chunks = K / PF_KC;

    // ---- which tile: (expert, BN-pair slab, row slab) -------------------------------------------------
    const int n_ntiles = a.n_ntiles;
    const int mt = blockIdx.x / n_ntiles, ni = blockIdx.x - mt * n_ntiles;
    // warp 0 looks the tile up, 32 experts per step: an expert with n pairs owns ceil(n / BN) consecutive tiles
    if (warp == 0) {
        int base = 0;
        bool found = false;
        for (int x0 = 0; x0 < a.n_experts && !found; x0 += 32) {
            const int x = x0 + lane;
            const int lo = x < a.n_experts ? a.grp_off[x] : 0, hi = x < a.n_experts ? a.grp_off[x + 1] : 0;
            const int nt = (hi - lo + BN - 1) / BN;
            int incl = nt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int t = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += t; }
            const bool hit = mt >= base + incl - nt && mt < base + incl;
            if (hit) { s_tile[0] = x; s_tile[1] = lo + (mt - (base + incl - nt)) * BN; s_tile[2] = hi; }
            found = __any_sync(0xffffffffu, hit);
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (!found && lane == 0) s_tile[0] = -1;
    }
    __syncthreads();
    const int e = s_tile[0], m0 = s_tile[1], m_end = s_tile[2];
    if (e < 0) return;                                        // grid is an upper bound on the tile count

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; s++) { pf_bar_init(&full_bar[s], 5); pf_bar_init(&empty_bar[s], PF_ISSUERS); }   // the copy's expect_tx arrival + four warps; one commit per issuer
        pf_bar_init(&accum_bar, PF_ISSUERS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PF_GROUPS * 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_u32(&s_tmem)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    if (tid == 0) TR(4003);

    if (warp < PF_GROUPS * 4) {
        // ================= producers: group g fills stage g for chunks g, g + 3, ... ======================
        const int group = warp >> 2, gtid = tid & 127;          // gtid = weight row of the tile = TMEM lane
        long long wrow; const uint8_t *wbase;
        if (MODE == MODE_GATEUP) { wrow = (long long)ni * NROW + (gtid & 63); wbase = gtid < 64 ? a.wa[e] : a.wb[e]; }
        else { wrow = (long long)ni * NROW + gtid; wbase = a.wa[e]; }
        const bool row_ok = wrow < a.out_f;
        const uint8_t *wunit = wbase + (row_ok ? (wrow >> 3) * nb * (long long)HTB : 0);
        const int rr = (int)(wrow & 7);
        // Q4_K: the 48 weight-block bytes of the NEXT chunk of this group are requested before waiting for the stage
        Q4Raw raw_next = {};
        if (QT == QT_Q4K && row_ok && group < n_chunks) load_q4k(wunit + (long long)(group >> 2) * HTB, rr, group & 3, raw_next);
        for (int c = group; c < n_chunks; c += PF_GROUPS) {
            const int s = c % STAGES;
            const Q4Raw raw = raw_next;
            if (QT == QT_Q4K && row_ok && c + PF_GROUPS < n_chunks) {
                const int cn = c + PF_GROUPS;
                load_q4k(wunit + (long long)(cn >> 2) * HTB, rr, cn & 3, raw_next);
            }
            TR(c * 4 + 0);
            if (c >= STAGES && !pf_bar_wait(&empty_bar[s], ((c / STAGES) - 1) & 1, &s_abort)) break;
            uint8_t *stage = smem + (size_t)s * STAGE_BYTES;
            TR(c * 4 + 1);
            if (gtid == 0) {                                   // activations: NL planes x BN pairs x 64 columns, by the copy engine
                pf_expect_tx(&full_bar[s], NL * X_PLANE);
#pragma unroll
                for (int b = 0; b < NL; b++) pf_tma_plane(stage + NWL * W_PLANE + b * X_PLANE, &xmap, c * PF_KC, b, m0, &full_bar[s]);
            }
            // weights: this thread's row, 64 columns as two halves of 32 (= the two K steps of the chunk)
            uint8_t *wdst = stage + (gtid >> 3) * 128 + (gtid & 7) * 16;
            if (QT == QT_Q6K && row_ok) {
                static_assert(QT != QT_Q6K || NWL == 5, "Q6_K tiles carry five weight digits");
                dequant64_q6k_store<W_PLANE>(wunit + (long long)(c >> 2) * HTB, rr, c & 3, a.fw, wdst);
            } else {
#pragma unroll
                for (int hsel = 0; hsel < 2; hsel++) {
                    uint32_t pl[NWL][8];
                    if (QT == QT_Q4K && row_ok) expand_q4k<NWL>(raw, c & 3, hsel, a.fw, pl);
                    else {
#pragma unroll
                        for (int l = 0; l < NWL; l++)
#pragma unroll
                            for (int w = 0; w < 8; w++) pl[l][w] = 0;
                    }
#pragma unroll
                    for (int l = 0; l < NWL; l++) {
                        *reinterpret_cast<uint4 *>(wdst + hsel * (W_PLANE / 2) + l * W_PLANE) = make_uint4(pl[l][0], pl[l][1], pl[l][2], pl[l][3]);
                        *reinterpret_cast<uint4 *>(wdst + hsel * (W_PLANE / 2) + l * W_PLANE + W_PLANE / 4) = make_uint4(pl[l][4], pl[l][5], pl[l][6], pl[l][7]);
                    }
                }
            }
            TR(c * 4 + 2);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> visible to the MMA
            __syncwarp();
            if (lane == 0) pf_bar_arrive(&full_bar[s]);
            TR(c * 4 + 3);
        }

        // ================= epilogue: TMEM lane = weight row, columns = pairs ================================
        if (pf_bar_wait(&accum_bar, 0, &s_abort)) {
            if ((tid & 127) == 0) TR(4000 + 10 * (tid >> 7));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
            int64_t *exch = reinterpret_cast<int64_t *>(smem) + group * 1024;     // gate/up: two buffers of [128 rows][4] per group (the stages are free now)
            int nl_max = 0, round = 0;
            for (int c0 = group * 8; c0 < BN; c0 += 8 * PF_GROUPS, round++) {     // the groups share the columns
                int64_t y[8];
                long long tok[8];
                int64_t gate[8];
                if (MODE == MODE_DOWN) {                       // requested before the accumulators are read, so the latencies overlap
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const long long pair = (long long)m0 + c0 + j;
                        const bool live = pair < m_end;
                        tok[j] = !live ? -1 : a.pair_tok ? a.pair_tok[pair] : pair;
                        gate[j] = live && a.gates ? a.gates[pair] : 0;
                    }
                }
                {
                    int r[NACC][8];
#pragma unroll
                    for (int s = 0; s < NACC; s++) pf_tmem_ld8(tlane + s * BN + c0, r[s]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 8; j++) y[j] = pf_recombine<NACC>(r, j, a.fw);
                }
                if (MODE == MODE_GATEUP) {
                    // gate rows keep columns 0..3 and hand 4..7 to their up row; up rows hand 0..3 to their gate row
                    const bool is_up = gtid >= 64;
                    int64_t *mine = exch + (round & 1) * 512 + gtid * 4, *theirs = exch + (round & 1) * 512 + (gtid ^ 64) * 4;
#pragma unroll
                    for (int j = 0; j < 4; j++) mine[j] = y[is_up ? j : 4 + j];
                    pf_group_sync(group);
                    const int jb = is_up ? 4 : 0;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const long long pair = (long long)m0 + c0 + jb + j;
                        const bool live = pair < m_end;               // predicated, not a break: the four chains interleave
                        const int64_t yg = is_up ? theirs[j] : y[j], yu = is_up ? y[4 + j] : theirs[j];
                        const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
                        const int64_t gu = mul_shift(sg, yu, a.fa);
                        bool ok;
                        const uint64_t d = balanced_digits8(gu, ok);
                        if (!live) continue;
                        if (!ok) atomicOr(a.flags, 1);
                        nl_max = max(nl_max, digits_used(d));
                        if (row_ok) {
                            if (a.out) a.out[pair * a.out_f + wrow] = gu;
                            int8_t *ol = a.out_limbs + pair * 8 * a.out_f + wrow;
#pragma unroll
                            for (int l = 0; l < 8; l++) ol[l * a.out_f] = (int8_t)(d >> (8 * l));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const long long pair = (long long)m0 + c0 + j;
                        if (pair >= m_end || !row_ok) continue;
                        if (MODE == MODE_LINEAR) a.out[pair * a.out_f + wrow] = y[j];
                        else atomicAdd(reinterpret_cast<unsigned long long *>(a.out + tok[j] * a.out_f + wrow),
                                       (unsigned long long)mul_shift(y[j], gate[j], a.fa));
                    }
                }
            }
            if (MODE == MODE_GATEUP && a.out_nl) {
                nl_max = max(nl_max, __shfl_xor_sync(0xffffffffu, nl_max, 16)); nl_max = max(nl_max, __shfl_xor_sync(0xffffffffu, nl_max, 8));
                nl_max = max(nl_max, __shfl_xor_sync(0xffffffffu, nl_max, 4));  nl_max = max(nl_max, __shfl_xor_sync(0xffffffffu, nl_max, 2));
                nl_max = max(nl_max, __shfl_xor_sync(0xffffffffu, nl_max, 1));
                if (lane == 0 && nl_max > 0) atomicMax(a.out_nl, nl_max);
            }
        }
        if ((tid & 127) == 0) TR(4001 + 10 * (tid >> 7));
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
        // ================= MMA issuers ===================================================================
        // One thread can only issue an MMA every few cycles and a chunk needs 2*NL*NWL of them, so the digit pairs
        // are split over three issuing warps by accumulator (s = a + b belongs to issuer s % 3: MMAs into
        // different accumulators are independent).  Descriptors are a per-stage base plus compile-time offsets.
        if (lane == 0) {
            constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(PF_BM >> 4) << 24);
            const int issuer = warp - PF_GROUPS * 4;
            bool ok = true;
            for (int c = 0; c < n_chunks && ok; c++) {
                const int s = c % STAGES;
                ok = pf_bar_wait(&full_bar[s], (c / STAGES) & 1, &s_abort);
                if (!ok) break;
                if (warp == PF_GROUPS * 4 && tron) d_tr[2048 + c * 2] = clock64();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t stage = pf_u32(smem + (size_t)s * STAGE_BYTES);
                const uint64_t dw0 = pf_desc(stage, W_PLANE / 4, 128), dx0 = pf_desc_sw64(stage + NWL * W_PLANE);
                const uint32_t later = c > 0 ? 1u : 0u;
                auto issue = [&](auto iss_c) {                 // ISS is a compile-time constant: the skipped pairs fold away
                    constexpr int ISS = decltype(iss_c)::value;
                    uint32_t seen = 0;
#pragma unroll
                    for (int ks = 0; ks < 2; ks++)
#pragma unroll
                        for (int b = 0; b < NL; b++)
#pragma unroll
                            for (int w = 0; w < NWL; w++) {
                                const int acc = b + w;
                                const bool first = !((seen >> acc) & 1u);
                                seen |= 1u << acc;
                                if (acc % PF_ISSUERS != ISS) continue;
                                const uint64_t dw = dw0 + (uint64_t)((w * W_PLANE + ks * (W_PLANE / 2)) >> 4);
                                const uint64_t dx = dx0 + (uint64_t)((b * X_PLANE + ks * 32) >> 4);
                                pf_mma(tmem + acc * BN, dw, dx, IDESC, first ? later : 1u);
                            }
                };
                if (issuer == 0) issue(std::integral_constant<int, 0>{});
                else if (issuer == 1) issue(std::integral_constant<int, 1>{});
                else issue(std::integral_constant<int, 2>{});
                if (warp == PF_GROUPS * 4 && tron) d_tr[2048 + c * 2 + 1] = clock64();
                pf_commit(&empty_bar[s]);                      // stage free once every issuer's MMAs have read it
            }
            if (ok) pf_commit(&accum_bar);                     // this issuer's MMAs done -> epilogue may read TMEM after all three
        }
        __syncwarp();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == PF_GROUPS * 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
    if (tid == 0 && s_abort) atomicOr(a.flags, 8);
}

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

template <int QT, int MODE, int NL, int NWL, int BN>
cudaError_t launch_pf(const PrefillArgs &a_in, cudaStream_t s, int shape) {
    __atomic_fetch_add(&g_prefill_launches[shape], 1ULL, __ATOMIC_RELAXED);
    PrefillArgs a = a_in;
    constexpr int W_PLANE = 2 * 2 * (PF_BM / 8) * 128, X_PLANE = BN * PF_KC;
    constexpr size_t smem = (size_t)pf_stages(NWL * W_PLANE + NL * X_PLANE) * (NWL * W_PLANE + NL * X_PLANE) + 1024;
    constexpr int NROW = MODE == MODE_GATEUP ? PF_BM / 2 : PF_BM;
    a.n_ntiles = (int)((a.out_f + NROW - 1) / NROW);
    a.sig_log2e = sigmoid_log2e(a.fa); a.sig_clip = sigmoid_clip(a.fa);
    const long long K = a.n_blocks * 256;
    // activation planes as a [rows][planes][K] byte tensor; rows reached through an index are gathered into pair order first
    const int8_t *planes = a.xl;
    long long n_planes = 8;
    if (a.xidx) {
        if (!a.xg) return cudaErrorInvalidValue;
        gather_planes_kernel<<<(unsigned)a.n_pairs, 128, 0, s>>>(a.xl, a.xidx, a.xg, (long long)NL * K, 8 * K, a.grp_off + a.n_experts);
        note_launch();
        planes = a.xg; n_planes = NL;
    }
    EncodeTiled enc = encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap map;
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)n_planes, (cuuint64_t)a.n_pairs};
    const cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)(n_planes * K)};
    const cuuint32_t box[3] = {PF_KC, 1, BN}, estr[3] = {1, 1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t *>(planes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel<QT, MODE, NL, NWL, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const long long max_mtiles = (a.n_pairs + BN - 1) / BN + a.n_experts;
    prefill_kernel<QT, MODE, NL, NWL, BN><<<(unsigned)(max_mtiles * a.n_ntiles), PF_THREADS, smem, s>>>(a, map);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

// nl: digits the activation needs (host-known upper bound).  Returns cudaErrorNotSupported when the
// combination has no tensor-core instantiation (the caller then uses the streamed kernels).
cudaError_t launch_prefill(int qtype, int mode, int nl, const PrefillArgs &a, cudaStream_t s) {
    if (a.n_blocks <= 0 || a.n_blocks * 256 > 8192 || a.out_f <= 0 || a.n_pairs <= 0) return cudaErrorInvalidValue;
    if (a.fw < 1 || a.fw > 32) return cudaErrorNotSupported;              // the epilogue's recombination floors the low group only
    if (qtype == QT_Q4K && mode == MODE_GATEUP) {
        if (nl <= 3) return launch_pf<QT_Q4K, MODE_GATEUP, 3, 4, 80>(a, s, 0);
        if (nl == 4) return launch_pf<QT_Q4K, MODE_GATEUP, 4, 4, 64>(a, s, 1);
    }
    if (qtype == QT_Q6K && mode == MODE_DOWN) {
        if (nl <= 5) return launch_pf<QT_Q6K, MODE_DOWN, 5, 5, 48>(a, s, 2);
        if (nl == 6) return launch_pf<QT_Q6K, MODE_DOWN, 6, 5, 48>(a, s, 3);
    }
    if (qtype == QT_Q4K && mode == MODE_DOWN) {
        if (nl <= 5) return launch_pf<QT_Q4K, MODE_DOWN, 5, 4, 64>(a, s, 4);
    }
    if (qtype == QT_Q4K && mode == MODE_LINEAR) {
        if (nl <= 3) return launch_pf<QT_Q4K, MODE_LINEAR, 3, 4, 64>(a, s, 5);
        if (nl <= 5) return launch_pf<QT_Q4K, MODE_LINEAR, 5, 4, 64>(a, s, 6);
    }
    return cudaErrorNotSupported;
}

}  // namespace iie
extern "C" void iie_pf_trace_block(int v, int mode) { cudaMemcpyToSymbol(iie::d_tr_block, &v, sizeof(int)); cudaMemcpyToSymbol(iie::d_tr_mode, &mode, sizeof(int)); }
extern "C" void iie_pf_trace_read(long long *out) { cudaMemcpyFromSymbol(out, iie::d_tr, sizeof(long long) * 4200); }
extern "C" void iie_pf_exp(int v) { cudaMemcpyToSymbol(iie::d_pf_exp, &v, sizeof(int)); }
