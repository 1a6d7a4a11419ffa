// Whole decode step of the MoE decoder as ONE persistent cooperative kernel: every block of the model
// (RMSNorm, fused Q/K/V product, rotation, cache append, exact softmax attention, O product, router product, top-k,
// sigmoid gates, gate/up with integer SiLU, down with gate-weighted combine, both added to the residual row) runs
// inside a single launch, one CTA per SM.
//
// Why one kernel.  At batch 1 a block moves ~52 MB (weights of the routed experts, attention matrices, visible cache
// rows) through about ten dependent steps.  As separate launches every step pays its own start-up (launch, first byte
// from HBM, drain) and HBM idles in between; measured, the six launches of a block took ~62 us for what is 8 us of
// traffic.  Here every CTA owns a fixed share of every step's bytes and a dedicated producer warp streams them, in the
// order they will be needed, through a ring of shared-memory slots with cp.async.bulk + mbarriers.  The ring runs
// ahead of the arithmetic across the step boundaries and across blocks (addresses of the attention matrices and the
// cache rows are known up front; the expert matrices become known when the routing of the block is done), so HBM
// stays busy while the consumer warps multiply, exchange softmax statistics or wait at a grid-wide barrier.
//
// Steps of a block and what crosses CTAs (all through global memory, L2-coherent loads, grid-wide arrive/wait
// counters; arrive and wait are separate so that independent work hides the latency of a barrier):
//   P0  h = rmsnorm(x) (every CTA, redundantly) -> digit planes in shared memory; [q|k|v] = h Wqkv^T and the router
//       logits: tiles of 16 rows dealt to the CTAs                                      -> arrive QKV
//   P1  wait QKV: top-k + gates (every CTA), expert pointers to the producer; rotate q; the first CTA of each KV head
//       rotates and appends the new key / value; scores of this CTA's key chunk, row maxima (atomicMax) -> arrive MAX
//       gate/up tiles of the routed experts, SiLU * up, digit planes of the product      -> arrive GU
//   P2  wait MAX: exponentials of the chunk, normaliser (atomicAdd)                      -> arrive Z
//       wait GU: down tiles, (y * gate) >> fa added to x (integer atomics: order-free)
//   P3  wait Z: probabilities x values of the chunk added to the per-head sums           -> arrive ACC
//   P4  wait ACC: digit planes of the attention output; O tiles added to x              -> arrive X (next block waits)
//
// Arithmetic is that of stream.cu / attn.cu / route.cu (same item code, same floors), so the bytes are those of the
// per-stage kernels and of north-mini-code/src/nmc/cohere2.py:357-376 (block_cached, m = 1).
//
// Every wait is bounded (mbarrier polls and barrier polls give up after a fixed count, raise flag bit 3 and make the
// remaining waits fall through); the producer waits for its own copies in flight before the CTA exits.  The launch is
// cooperative: all CTAs are resident, which the grid-wide counters rely on.
#include <cooperative_groups.h>

#include "kernels.h"
#include "layout.cuh"
#include "mma_items.cuh"
#include "norm.cuh"

namespace iie {

namespace {

constexpr int DK_CW = 16;                       // consumer warps
constexpr int DK_CT = DK_CW * 32;               // consumer threads
constexpr int DK_THREADS = DK_CT + 32;          // plus the producer warp
constexpr int DK_NS = 7;                        // ring slots
constexpr int DK_SLOT = 20160;                  // bytes per slot: a Q4_K 16-row x 8-block tile (18432) or two Q6_K 16-row x 3-block tiles
constexpr int DK_KSLOTS = 3;                    // ring slots one key (or value) chunk may take
constexpr int DK_PAD = 32;                      // padding of a digit plane (bytes): planes start on different banks
constexpr int DK_EPT = 4;                       // residual-row elements per consumer thread (d_model <= 2048)
constexpr int DK_MAXREP = 8;                    // query heads per KV head
constexpr int DK_MAXK = 64;                     // routed experts per token
constexpr unsigned DK_POLLS = 1u << 22;
constexpr int DK_SMEM_MAX = 227 * 1024 - 4096;   // dynamic shared memory: the 227 KB of a CTA less this kernel's static arrays
enum { GB_QKV = 0, GB_MAX, GB_GU, GB_Z, GB_ACC, GB_X, GB_COUNT };
enum { KIND_P0 = 0, KIND_G, KIND_D, KIND_O };

__device__ __forceinline__ uint32_t dk_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(DK_CT) : "memory"); }   // consumer warps only

// Everything the warps of a CTA share lives in shared memory (one copy per CTA, broadcast reads), never in per-thread
// structures: a per-thread copy would sit in local memory, and with 200+ KB of shared memory in use the L1 left for
// local memory is a few tens of KB.
struct Geo {
    int nb, nbo, nbd;                 // 256-column blocks of d_model, of n_heads*head_dim, of e_ffn
    int t_qkv, t_r, n_p0;             // 16-row tiles of Wqkv and of the router; together
    int nht_g, n_g;                   // 8-row units of one expert's gate (= up) matrix; gate/up tiles of all routed experts
    int td, TD, ipe, n_d;             // down: tiles per expert, tiles per ring item, items per expert, items of all routed experts
    int to, okn;                      // O: row tiles; ring slots per tile (K chunks of <= 8 blocks)
    int htb_d;                        // bytes of a down unit block
    int cpk, kps;                     // CTAs per KV head, keys per ring slot
};

struct Shared {
    uint64_t full[DK_NS], empty[DK_NS], idsbar;           // mbarriers
    Geo g;
    uint8_t *slots;
    unsigned long long *red;                              // [DK_NS][2][128]
    int done[DK_NS * 2], slot_done[DK_NS];                // blocks of each tile already added; tiles of each item finished
    int ids[DK_MAXK];
    int64_t gates[DK_MAXK];
    const uint8_t *sel[3 * DK_MAXK];
    unsigned long long lo[DK_CW], hi[DK_CW], mx[DK_CW], gmx[DK_CW];
    unsigned long long rms, inv, gm;
    long long hmax[DK_MAXREP];
    unsigned long long z[DK_MAXREP];
    int bad, nl, abort;
};

__device__ __forceinline__ bool mb_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(dk_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded, abort-aware wait: false when the phase never completed (the caller skips the work that needed it).
__device__ __forceinline__ bool mb_wait(uint64_t *bar, uint32_t parity, int *abort_ptr) {
    volatile int *abort_flag = abort_ptr;
    for (unsigned it = 0; it < DK_POLLS; it++) {
        if (mb_try(bar, parity)) return true;
        if ((it & 255) == 255 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void mb_arrive(uint64_t *bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dk_u32(bar)) : "memory"); }
__device__ __forceinline__ void mb_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(dk_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dk_bulk(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dk_u32(dst)), "l"(src), "r"(bytes), "r"(dk_u32(bar)) : "memory");
}

// ---- grid-wide counters: one arrival per CTA per block ---------------------------------------------------------------
__device__ __forceinline__ void grid_arrive(unsigned *bars, int id) {          // one thread, after cbar()
    __threadfence();
    atomicAdd(bars + id, 1u);
}
__device__ __forceinline__ void grid_wait(unsigned *bars, int id, unsigned target, int *abort_ptr) {   // one thread
    volatile int *abort_flag = abort_ptr;
    for (unsigned it = 0; it < DK_POLLS; it++) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bars + id) : "memory");
        if (v >= target) { __threadfence(); return; }
        if (*abort_flag) return;
        __nanosleep(32);
    }
    *abort_flag = 1;
}

// ---- geometry shared by the producer and the consumers ------------------------------------------------------------------
__device__ __forceinline__ Geo make_geo(const DecodeArgs &a, int down_q) {
    Geo g;
    g.nb = a.d / 256; g.nbo = a.H * a.hd / 256; g.nbd = a.eff / 256;
    const int nht_qkv = (a.H + 2 * a.Hkv) * a.hd / 8, nht_r = (a.E + 7) / 8;
    g.t_qkv = (nht_qkv + 1) / 2; g.t_r = (nht_r + 1) / 2; g.n_p0 = g.t_qkv + g.t_r;
    g.nht_g = a.eff / 8; g.n_g = a.k * g.nht_g;
    g.htb_d = down_q == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    g.td = (a.d / 8 + 1) / 2;
    g.TD = DK_SLOT / (2 * g.nbd * g.htb_d) >= 2 ? 2 : 1;
    g.ipe = (g.td + g.TD - 1) / g.TD; g.n_d = a.k * g.ipe;
    g.to = g.td; g.okn = (g.nbo + 7) / 8;
    g.cpk = (int)gridDim.x / a.Hkv; g.kps = DK_SLOT / (a.hd * 4);
    return g;
}

// contiguous share of n items for CTA c of nc
__device__ __forceinline__ void share(int n, int c, int nc, int &lo, int &hi) {
    lo = (int)((long long)n * c / nc); hi = (int)((long long)n * (c + 1) / nc);
}

// this CTA's key chunk: KV head, first key, keys (history only; the new token's key is handled apart by chunk 0)
struct Chunk { int kv, ci, k0, nk, slots; bool active, owner; };

__device__ __forceinline__ Chunk make_chunk(const DecodeArgs &a, const Geo &g, long long pos, long long lo) {
    Chunk ch;
    const int c = (int)blockIdx.x;
    ch.active = c < g.cpk * a.Hkv;
    ch.kv = ch.active ? c / g.cpk : 0; ch.ci = ch.active ? c % g.cpk : 0;
    const long long n_hist = pos - lo, per = (n_hist + g.cpk - 1) / g.cpk;
    const long long k0 = lo + (long long)ch.ci * per, k1 = min(k0 + per, pos);
    ch.k0 = (int)k0; ch.nk = ch.active ? (int)max(0LL, k1 - k0) : 0;
    ch.slots = (ch.nk + g.kps - 1) / g.kps;
    ch.owner = ch.active && ch.ci == 0;
    return ch;
}

// ---- the producer: one lane streams every item of this CTA through the ring, in consumption order ----------------------
struct Producer {
    Shared *sh;
    unsigned seq, used_mask, parity_mask;                  // per slot: ever used; parity of its last request

    __device__ __forceinline__ bool acquire(int &slot) {
        slot = (int)(seq % DK_NS);
        if (*(volatile int *)&sh->abort) return false;
        if (seq >= DK_NS && !mb_wait(&sh->empty[slot], ((seq / DK_NS) - 1) & 1, &sh->abort)) return false;
        return true;
    }
    __device__ __forceinline__ void commit(int slot) {
        used_mask |= 1u << slot;
        parity_mask = (parity_mask & ~(1u << slot)) | (((seq / DK_NS) & 1u) << slot);
        seq++;
    }
    __device__ __forceinline__ bool one(const void *src, uint32_t bytes) {
        int slot;
        if (!acquire(slot)) return false;
        mb_expect(&sh->full[slot], bytes);
        dk_bulk(sh->slots + (size_t)slot * DK_SLOT, src, bytes, &sh->full[slot]);
        commit(slot);
        return true;
    }
    __device__ __forceinline__ bool two(const void *s0, const void *s1, uint32_t bytes_each) {
        int slot;
        if (!acquire(slot)) return false;
        mb_expect(&sh->full[slot], 2 * bytes_each);
        uint8_t *dst = sh->slots + (size_t)slot * DK_SLOT;
        dk_bulk(dst, s0, bytes_each, &sh->full[slot]);
        dk_bulk(dst + bytes_each, s1, bytes_each, &sh->full[slot]);
        commit(slot);
        return true;
    }
};

__device__ __noinline__ void producer_run(const DecodeArgs &a, Shared *sh, long long pos) {
    Producer p;
    p.sh = sh; p.seq = 0; p.used_mask = 0; p.parity_mask = 0;
    const int c = (int)blockIdx.x, nc = (int)gridDim.x;
    const Geo g = sh->g;
    bool ok = true;
    for (int L = 0; L < a.n_layers && ok; L++) {
        const DecodeLayer &ly = a.layers[L];
        const long long lo = (!ly.full && a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        const Chunk ch = make_chunk(a, g, pos, lo);
        int i0, i1;
        // P0 tiles: rows of Wqkv, then of the router
        share(g.n_p0, c, nc, i0, i1);
        for (int i = i0; i < i1 && ok; i++) {
            const bool r = i >= g.t_qkv;
            const int tile = r ? i - g.t_qkv : i, n_ht = r ? (a.E + 7) / 8 : (a.H + 2 * a.Hkv) * a.hd / 8;
            const uint8_t *w = r ? ly.router : ly.wqkv;
            const int units = (2 * tile + 1 < n_ht) ? 2 : 1;
            ok = p.one(w + (size_t)(2 * tile) * g.nb * HTB_Q4K, (uint32_t)(units * g.nb * HTB_Q4K));
        }
        // keys of this CTA's chunk
        for (int j = 0; j < ch.slots && ok; j++) {
            const int n = min(g.kps, ch.nk - j * g.kps);
            ok = p.one(ly.kcache + ((size_t)ch.kv * a.Lmax + ch.k0 + (size_t)j * g.kps) * a.hd, (uint32_t)(n * a.hd * 4));
        }
        // routed experts: their pointers arrive from the consumers once the routing of this block is known
        share(g.n_g, c, nc, i0, i1);
        int d0, d1;
        share(g.n_d, c, nc, d0, d1);
        if (ok && (i1 > i0 || d1 > d0)) ok = mb_wait(&sh->idsbar, (uint32_t)(L & 1), &sh->abort);
        for (int i = i0; i < i1 && ok; i++) {
            const int s = i / g.nht_g, u = i - s * g.nht_g;
            ok = p.two(sh->sel[s] + (size_t)u * g.nb * HTB_Q4K, sh->sel[a.k + s] + (size_t)u * g.nb * HTB_Q4K, (uint32_t)(g.nb * HTB_Q4K));
        }
        for (int i = d0; i < d1 && ok; i++) {
            const int s = i / g.ipe, q = i - s * g.ipe;
            const int n_ht = a.d / 8, units = min(2 * g.TD, n_ht - 2 * q * g.TD);
            ok = p.one(sh->sel[2 * a.k + s] + (size_t)(2 * q * g.TD) * g.nbd * g.htb_d, (uint32_t)(units * g.nbd * g.htb_d));
        }
        // values of the chunk
        for (int j = 0; j < ch.slots && ok; j++) {
            const int n = min(g.kps, ch.nk - j * g.kps);
            ok = p.one(ly.vcache + ((size_t)ch.kv * a.Lmax + ch.k0 + (size_t)j * g.kps) * a.hd, (uint32_t)(n * a.hd * 4));
        }
        // O tiles: one ring slot per chunk of 8 K-blocks; the two 8-row units of a tile lie nbo blocks apart
        share(g.to, c, nc, i0, i1);
        for (int i = i0; i < i1 && ok; i++)
            for (int kc = 0; kc < g.okn && ok; kc++) {
                const int nbk = min(8, g.nbo - kc * 8);
                const uint8_t *u0 = ly.wo + ((size_t)(2 * i) * g.nbo + (size_t)kc * 8) * HTB_Q4K;
                ok = p.two(u0, u0 + (size_t)g.nbo * HTB_Q4K, (uint32_t)(nbk * HTB_Q4K));
            }
    }
    // copies of this lane still in flight must land before the CTA's shared memory goes away
    for (int s = 0; s < DK_NS; s++)
        if ((p.used_mask >> s) & 1u) {
            for (unsigned it = 0; it < DK_POLLS; it++)
                if (mb_try(&sh->full[s], (p.parity_mask >> s) & 1u)) break;
        }
}

// ---- consumers: 16-row tiles of a ring item on the warp MMA, K split over the warps -------------------------------------
// Epilogue of one finished tile: lanes 0..15 own its 16 rows (gate/up: lanes 0..7 own the 8 (gate, up) row pairs).
__device__ __forceinline__ void tile_epilogue(const DecodeArgs &a, const Shared *sh, int kind, int gi, int tile_in_item,
                                              const volatile unsigned long long *rv, int lane) {
    const Geo &g = sh->g;
    if (kind == KIND_P0) {
        const bool r = gi >= g.t_qkv;
        const int tile = r ? gi - g.t_qkv : gi;
        const long long row = (long long)tile * 16 + lane, rows = r ? a.E : (long long)(a.H + 2 * a.Hkv) * a.hd;
        if (lane < 16 && row < rows) {
            unsigned long long cc[8];
#pragma unroll
            for (int c = 0; c < 8; c++) cc[c] = rv[lane * 8 + c];
            (r ? a.logits : a.qkv)[row] = recombine_cols(cc, a.fw);
        }
    } else if (kind == KIND_G) {
        const int s = gi / g.nht_g, u = gi - s * g.nht_g;
        if (lane < 8) {
            unsigned long long cg[8], cu[8];
#pragma unroll
            for (int c = 0; c < 8; c++) { cg[c] = rv[lane * 8 + c]; cu[c] = rv[(lane + 8) * 8 + c]; }
            const int64_t yg = recombine_cols(cg, a.fw), yu = recombine_cols(cu, a.fw);
            const int64_t sg = mul_shift(yg, sigmoid_fixed_c(yg, a.fa, a.sig_log2e, a.sig_clip), a.fa);
            const int64_t gu = mul_shift(sg, yu, a.fa);
            bool ok;
            const uint64_t dg = balanced_digits8(gu, ok);
            if (!ok) atomicOr(a.flags, 1);
            const long long row = (long long)u * 8 + lane;
#pragma unroll
            for (int l = 0; l < 8; l++) a.gul[((long long)s * 8 + l) * a.eff + row] = (int8_t)(dg >> (8 * l));
        }
    } else if (kind == KIND_D) {
        const int s = gi / g.ipe, q = gi - s * g.ipe;
        const long long row = ((long long)q * g.TD + tile_in_item) * 16 + lane;
        if (lane < 16 && row < a.d) {
            unsigned long long cc[8];
#pragma unroll
            for (int c = 0; c < 8; c++) cc[c] = rv[lane * 8 + c];
            const int64_t y = recombine_cols(cc, a.fw);
            atomicAdd(reinterpret_cast<unsigned long long *>(a.x + row), (unsigned long long)mul_shift(y, sh->gates[s], a.fa));
        }
    } else {
        const long long row = (long long)gi * 16 + lane;
        if (lane < 16 && row < a.d) {
            unsigned long long cc[8];
#pragma unroll
            for (int c = 0; c < 8; c++) cc[c] = rv[lane * 8 + c];
            atomicAdd(reinterpret_cast<unsigned long long *>(a.x + row), (unsigned long long)recombine_cols(cc, a.fw));
        }
    }
}

// Multiply the items [i0, i1) of `kind`, whose first ring sequence number is seq0: (tile, block) pairs are dealt to the
// warps, partial sums meet in `red`, the warp that completes a tile runs its epilogue and, when that was the item's
// last tile, hands the item's slots back to the producer.  An item is one slot holding one tile (P0, gate/up), one slot
// holding up to two tiles (down), or one tile whose K blocks span several slots (O).
template <int QT>
__device__ __noinline__ void lin_items(const DecodeArgs &a, Shared *sh, int kind, int i0, int i1, unsigned seq0, bool half,
                                       const int8_t *planes, int pstride) {
    constexpr int HTB = QT == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t = lane & 3;
    uint32_t bf[16];
    int bcur = -1;
    int widx = 0;                                           // (tile, block) pairs of the earlier items: keeps the deal round-robin
    const int sp = kind == KIND_O ? sh->g.okn : 1;          // ring slots per item
    for (int i = i0; i < i1; i++) {
        int tiles = 1, nbk = sh->g.nb, n_units = 2;
        if (kind == KIND_P0) {
            const bool r = i >= sh->g.t_qkv;
            const int tile = r ? i - sh->g.t_qkv : i, n_ht = r ? (a.E + 7) / 8 : (a.H + 2 * a.Hkv) * a.hd / 8;
            n_units = (2 * tile + 1 < n_ht) ? 2 : 1;
        } else if (kind == KIND_D) {
            const int q = i % sh->g.ipe;
            nbk = sh->g.nbd;
            tiles = min(sh->g.TD, sh->g.td - q * sh->g.TD);
            n_units = min(2 * sh->g.TD, a.d / 8 - 2 * q * sh->g.TD);
        } else if (kind == KIND_O) {
            nbk = sh->g.nbo;
        }
        const unsigned first = seq0 + (unsigned)(i - i0) * (unsigned)sp;
        const int slot0 = (int)(first % DK_NS);
        const int n_work = tiles * nbk;
        for (int w = ((warp - widx % DK_CW) + DK_CW) % DK_CW; w < n_work; w += DK_CW) {
            const int tj = w / nbk, b = w - tj * nbk;
            const int sj = kind == KIND_O ? b >> 3 : 0, bl = kind == KIND_O ? b & 7 : b;
            const int bps = kind == KIND_O ? min(8, nbk - sj * 8) : nbk;     // blocks of one unit inside this slot
            const unsigned sq = first + (unsigned)sj;
            const int slot = (int)(sq % DK_NS);
            // warp-uniform outcome: the MMA below needs every lane
            if (!__all_sync(0xffffffffu, mb_wait(&sh->full[slot], (sq / DK_NS) & 1, &sh->abort))) break;
            if (b != bcur) { load_bfrag<QT, false>(planes + col_limb(gq) * pstride + b * 256, t, bf); bcur = b; }
            const uint8_t *sb = sh->slots + (size_t)slot * DK_SLOT;
            const uint8_t *ua = sb + (size_t)(2 * tj) * bps * HTB + (size_t)bl * HTB;
            const uint8_t *ub = (2 * tj + 1 < n_units) ? ua + (size_t)bps * HTB : ua;
            int64_t acc[4] = {0, 0, 0, 0};
            run_item<QT, true>(ua, ub, lane, a.fw, bf, half, acc);
            unsigned long long *r = sh->red + ((size_t)slot0 * 2 + tj) * 128;
            atomicAdd(&r[gq * 8 + 2 * t], (unsigned long long)acc[0]);
            atomicAdd(&r[(gq + 8) * 8 + 2 * t], (unsigned long long)acc[2]);
            if (!half) {
                atomicAdd(&r[gq * 8 + 2 * t + 1], (unsigned long long)acc[1]);
                atomicAdd(&r[(gq + 8) * 8 + 2 * t + 1], (unsigned long long)acc[3]);
            }
            __threadfence_block();
            int prior = 0;
            if (lane == 0) prior = atomicAdd(&sh->done[slot0 * 2 + tj], 1);
            prior = __shfl_sync(0xffffffffu, prior, 0);
            if (prior != nbk - 1) continue;
            // last block of the tile: epilogue, then leave the accumulators clean for the slot's next use
            __threadfence_block();
            tile_epilogue(a, sh, kind, i, tj, r, lane);
            __syncwarp();
            for (int z = lane; z < 128; z += 32) r[z] = 0ULL;
            if (lane == 0) sh->done[slot0 * 2 + tj] = 0;
            __threadfence_block();
            int fin = 0;
            if (lane == 0) fin = atomicAdd(&sh->slot_done[slot0], 1);
            fin = __shfl_sync(0xffffffffu, fin, 0);
            if (fin == tiles - 1 && lane == 0) {
                sh->slot_done[slot0] = 0;
                for (int q = 0; q < sp; q++) mb_arrive(&sh->empty[(first + (unsigned)q) % DK_NS]);
            }
        }
        widx += n_work;
    }
}

// h = rmsnorm(x) * gain as balanced digit planes in shared memory; returns through sh->nl the digits in use.
__device__ __noinline__ void norm_planes(const DecodeArgs &a, Shared *sh, const int64_t *gain, int8_t *planes, int pstride) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, c = (int)blockIdx.x;
    int64_t xv[DK_EPT], gv[DK_EPT];
    u128 ssq = 0; unsigned long long mx = 0, gmx = 0;
    const int i0 = tid * DK_EPT;
#pragma unroll
    for (int e = 0; e < DK_EPT; e++) {
        const bool in = i0 + e < a.d;
        xv[e] = in ? __ldcg(a.x + i0 + e) : 0;
        gv[e] = in ? __ldg(gain + i0 + e) : 0;
        const unsigned long long v = uabs64(xv[e]), gg = uabs64(gv[e]);
        ssq += (u128)v * v; mx = v > mx ? v : mx; gmx = gg > gmx ? gg : gmx;
    }
    unsigned long long slo = (unsigned long long)ssq, shi = (unsigned long long)(ssq >> 64);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const unsigned long long lo2 = __shfl_xor_sync(0xffffffffu, slo, s), hi2 = __shfl_xor_sync(0xffffffffu, shi, s);
        const u128 sum = (((u128)shi << 64) | slo) + (((u128)hi2 << 64) | lo2);
        slo = (unsigned long long)sum; shi = (unsigned long long)(sum >> 64);
        const unsigned long long m2 = __shfl_xor_sync(0xffffffffu, mx, s), g2 = __shfl_xor_sync(0xffffffffu, gmx, s);
        mx = m2 > mx ? m2 : mx; gmx = g2 > gmx ? g2 : gmx;
    }
    if (lane == 0) { sh->lo[warp] = slo; sh->hi[warp] = shi; sh->mx[warp] = mx; sh->gmx[warp] = gmx; }
    if (tid == 0) { sh->bad = 0; sh->nl = 1; }
    cbar();
    if (tid == 0) {
        u128 total = 0; unsigned long long m = 0, gm = 0;
        for (int i = 0; i < DK_CW; i++) {
            total += ((u128)sh->hi[i] << 64) | sh->lo[i];
            m = sh->mx[i] > m ? sh->mx[i] : m; gm = sh->gmx[i] > gm ? sh->gmx[i] : gm;
        }
        if (m > (1ULL << 57)) sh->bad = 1;                 // keeps the 128-bit sum of squares exact
        u128 mean;
        if ((a.d & (a.d - 1)) == 0) mean = total >> (31 - __clz(a.d));
        else if ((total >> 64) == 0) mean = (u128)((unsigned long long)total / (unsigned long long)a.d);
        else mean = total / (u128)(unsigned long long)a.d;
        const u128 rms = isqrt128(mean + a.eps);
        if (rms == 0 || rms > (u128)0xFFFFFFFFFFFFFFFFULL) sh->bad = 1;
        sh->rms = (unsigned long long)rms; sh->gm = gm;
        sh->inv = rms != 0 ? 0xFFFFFFFFFFFFFFFFULL / (unsigned long long)rms : 0;
    }
    cbar();
    const unsigned long long rms = sh->rms, inv = sh->inv, gm = sh->gm;
    const bool dead = sh->bad != 0;                        // the row cannot be normalised exactly: zeros, flag raised
    bool bad = false, over = false;
    int nl = 1;
    uint32_t pw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < DK_EPT; e++) {
        int64_t y = 0;
        if (!dead && i0 + e < a.d) {
            if (uabs64(xv[e]) < (1ULL << (62 - a.fa)) && rms < (1ULL << 62)) y = floor_div_recip(xv[e] * ((long long)1 << a.fa), rms, inv);
            else {
                const i128 num = (i128)xv[e] * ((i128)1 << a.fa);
                i128 q = num / (i128)rms;
                if (num < 0 && q * (i128)rms != num) q -= 1;
                if (q > (i128)INT64_MAX || q < (i128)INT64_MIN) { bad = true; q = 0; }
                y = (int64_t)q;
            }
            if ((u128)uabs64(y) * gm > (u128)INT64_MAX) bad = true;      // the oracle refuses such a gain product
            y = mul_shift(y, gv[e], a.fa);
        }
        bool ok;
        const uint64_t dg = balanced_digits8(y, ok);
        over |= !ok;
        nl = max(nl, digits_used(dg));
#pragma unroll
        for (int l = 0; l < 8; l++) pw[l] |= (uint32_t)((dg >> (8 * l)) & 0xFF) << (8 * e);
    }
    if (i0 < a.d) {
#pragma unroll
        for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * pstride + i0) = pw[l];
    }
    if ((bad || dead) && c == 0) atomicOr(a.flags, 2);
    if (over && c == 0) atomicOr(a.flags, 1);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, s));
    if (lane == 0) atomicMax(&sh->nl, nl);
    cbar();
}

}  // namespace

__global__ void __launch_bounds__(DK_THREADS, 1) decode_kernel(const __grid_constant__ DecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) Shared sh_;
    Shared *sh = &sh_;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = (int)blockIdx.x, nc = (int)gridDim.x;
    // ---- the position: refuse (uniformly over the grid) a cell beyond what the host sized the launch for -------------------
    const long long pos = a.pos_dev ? (long long)*a.pos_dev : a.pos_bound;
    if (pos < 0 || pos > a.pos_bound || pos >= a.Lmax) {
        if (tid == 0 && c == 0) atomicOr(a.flags, 16);
        return;
    }
    // ---- shared-memory layout (offsets computed by the host the same way) -------------------------------------------------------
    uint8_t *slots = smem;
    unsigned long long *red = reinterpret_cast<unsigned long long *>(smem + (size_t)DK_NS * DK_SLOT);
    int8_t *planes = reinterpret_cast<int8_t *>(red + DK_NS * 2 * 128);
    const int pk = max(a.d, a.H * a.hd), pstride = pk + DK_PAD;
    int8_t *gup = planes + (size_t)8 * pstride;
    const int gstride = a.eff + DK_PAD;
    long long *s_sc = reinterpret_cast<long long *>(gup + (size_t)8 * gstride);                 // [keys][rep] scores; first the router logits
    const int maxkeys = DK_KSLOTS * (DK_SLOT / (a.hd * 4)) + 1, rep = a.H / a.Hkv;
    const int sc_elems = (max(maxkeys * rep, a.E) + 1) & ~1;                                   // every region starts on 16 bytes (vector loads)
    unsigned *s_e = reinterpret_cast<unsigned *>(s_sc + sc_elems);                             // [keys][rep] exponentials, then probabilities
    int32_t *s_q = reinterpret_cast<int32_t *>(s_e + ((maxkeys * rep + 3) & ~3));              // [rep][hd] rotated query heads
    int32_t *s_knew = s_q + rep * a.hd, *s_vnew = s_knew + a.hd;                               // the new token's key / value row

    if (tid == 0) {
        for (int s = 0; s < DK_NS; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dk_u32(&sh->full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dk_u32(&sh->empty[s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dk_u32(&sh->idsbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        sh->abort = 0; sh->slots = slots; sh->red = red;
        sh->g = make_geo(a, a.layers[0].down_q);
    }
    for (int i = tid; i < DK_NS * 2 * 128; i += DK_THREADS) red[i] = 0ULL;
    for (int i = tid; i < DK_NS * 2; i += DK_THREADS) sh->done[i] = 0;
    for (int i = tid; i < DK_NS; i += DK_THREADS) sh->slot_done[i] = 0;
    __syncthreads();

    if (warp == DK_CW) {                                     // ================= producer warp =================
        if (lane == 0) producer_run(a, sh, pos);
        __syncwarp();
        if (lane == 0 && sh->abort) atomicOr(a.flags, 8);
        return;
    }

    // ===================================== consumer warps =====================================
    unsigned seq = 0;                                        // ring sequence number of this CTA's next item
    const int half_hd = a.hd / 2;
    const int cpk = sh->g.cpk, kps = sh->g.kps;

    for (int L = 0; L < a.n_layers; L++) {
        const DecodeLayer &ly = a.layers[L];
        const int par = L & 1;
        const bool full = ly.full != 0;
        const long long lo = (!full && a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        // this CTA's key chunk (make_chunk, kept in scalars)
        const bool active = c < cpk * a.Hkv;
        const int kv = active ? c / cpk : 0, ci = active ? c % cpk : 0;
        const long long n_hist = pos - lo, per = (n_hist + cpk - 1) / cpk;
        const long long ck0 = lo + (long long)ci * per, ck1 = min(ck0 + per, pos);
        const int nk = active ? (int)max(0LL, ck1 - ck0) : 0, kslots = (nk + kps - 1) / kps;
        const bool owner = active && ci == 0;
        const unsigned target = (unsigned)(L + 1) * (unsigned)nc;
        long long *hmax = a.hmax + par * a.H;
        unsigned long long *Z = a.Z + par * a.H;
        long long *acc = a.acc + (long long)par * a.H * a.hd;

        // ================================ P0: RMSNorm, Q/K/V and router rows ================================
        if (L > 0) { if (tid == 0) grid_wait(a.bars, GB_X, (unsigned)L * (unsigned)nc, &sh->abort); cbar(); }
        if (c == 0) {                                        // statistics of the NEXT block (and, first of all, of this one)
            for (int pp = (L == 0 ? 0 : 1); pp < 2; pp++) {
                const int q = (par + pp) & 1;
                for (int i = tid; i < a.H; i += DK_CT) { a.hmax[q * a.H + i] = INT64_MIN; a.Z[q * a.H + i] = 0ULL; }
                for (int i = tid; i < a.H * a.hd; i += DK_CT) a.acc[(long long)q * a.H * a.hd + i] = 0;
            }
        }
        norm_planes(a, sh, ly.gain, planes, pstride);
        const bool half_h = sh->nl <= 4;
        int i0, i1;
        share(sh->g.n_p0, c, nc, i0, i1);
        lin_items<QT_Q4K>(a, sh, KIND_P0, i0, i1, seq, half_h, planes, pstride);
        seq += (unsigned)(i1 - i0);
        cbar();
        if (tid == 0) { grid_arrive(a.bars, GB_QKV); grid_wait(a.bars, GB_QKV, target, &sh->abort); }
        cbar();

        // ================================ P1: routing, scores, gate/up ================================
        {
            long long *lg = s_sc;                               // router logits, then reused for the scores
            for (int i = tid; i < a.E; i += DK_CT) lg[i] = __ldcg(a.logits + i);
            cbar();
            for (int e = tid; e < a.E; e += DK_CT) {
                const long long v = lg[e];
                int rank = 0;
                for (int j = 0; j < a.E; j++) { const long long w = lg[j]; rank += (w > v) || (w == v && j < e); }
                if (rank < a.k) {
                    sh->ids[rank] = e; sh->gates[rank] = sigmoid_fixed_c(v, a.fa, a.sig_log2e, a.sig_clip);
                    for (int m = 0; m < 3; m++) sh->sel[m * a.k + rank] = ly.tabs[(size_t)m * a.E + e];
                    if (c == 0 && a.ids_out) { a.ids_out[(long long)L * a.k + rank] = e; a.gates_out[(long long)L * a.k + rank] = sh->gates[rank]; }
                }
            }
            cbar();
            if (tid == 0) mb_arrive(&sh->idsbar);               // the producer may now request this block's expert tiles
        }
        // rotated query heads of this CTA's KV head; the chunk-0 CTA also rotates and appends the new key / value
        if (active) {
            const long long qoff = (long long)kv * rep * a.hd;
            bool wide = false;
            for (int idx = tid; idx < rep * half_hd; idx += DK_CT) {
                const int r = idx / half_hd, i = idx - r * half_hd;
                const int e0 = 2 * i, e1 = e0 + 1;                  // interleaved pairs (cohere2.py:114-120)
                int64_t x0 = __ldcg(a.qkv + qoff + r * a.hd + e0), x1 = __ldcg(a.qkv + qoff + r * a.hd + e1);
                if (!full) {
                    const int64_t cs = a.cos[pos * half_hd + i], sn = a.sin[pos * half_hd + i];
                    const int64_t y0 = (x0 * cs - x1 * sn) >> a.fa, y1 = (x0 * sn + x1 * cs) >> a.fa;
                    x0 = y0; x1 = y1;
                }
                s_q[r * a.hd + e0] = (int32_t)x0; s_q[r * a.hd + e1] = (int32_t)x1;
                wide |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
            }
            if (wide) atomicOr(a.flags, 32);                     // a query value beyond int32: this kernel cannot hold it
            if (owner) {
                const long long koff = (long long)a.H * a.hd + (long long)kv * a.hd, voff = koff + (long long)a.Hkv * a.hd;
                bool badkv = false;
                for (int i = tid; i < half_hd; i += DK_CT) {
                    int64_t x0 = __ldcg(a.qkv + koff + 2 * i), x1 = __ldcg(a.qkv + koff + 2 * i + 1);
                    if (!full) {
                        const int64_t cs = a.cos[pos * half_hd + i], sn = a.sin[pos * half_hd + i];
                        const int64_t y0 = (x0 * cs - x1 * sn) >> a.fa, y1 = (x0 * sn + x1 * cs) >> a.fa;
                        x0 = y0; x1 = y1;
                    }
                    badkv |= x0 != (int32_t)x0 || x1 != (int32_t)x1;
                    s_knew[2 * i] = (int32_t)x0; s_knew[2 * i + 1] = (int32_t)x1;
                    int32_t *dst = ly.kcache + ((long long)kv * a.Lmax + pos) * a.hd;
                    dst[2 * i] = (int32_t)x0; dst[2 * i + 1] = (int32_t)x1;
                }
                for (int i = tid; i < a.hd; i += DK_CT) {
                    const int64_t v = __ldcg(a.qkv + voff + i);
                    badkv |= v != (int32_t)v;
                    s_vnew[i] = (int32_t)v;
                    ly.vcache[((long long)kv * a.Lmax + pos) * a.hd + i] = (int32_t)v;
                }
                if (badkv) atomicOr(a.flags, 4);
            }
            if (tid < DK_MAXREP) { sh->hmax[tid] = INT64_MIN; sh->z[tid] = 0ULL; }
        }
        cbar();
        const int nk_all = nk + (owner ? 1 : 0);                 // keys this CTA scores: its history chunk, plus the new one
        const unsigned kseq = seq;                               // ring items of the key chunk
        if (active) {
            bool ready = true;
            for (int j = 0; j < kslots; j++)
                ready = mb_wait(&sh->full[(kseq + j) % DK_NS], ((kseq + j) / DK_NS) & 1, &sh->abort) && ready;
            const int npair = (rep + 1) / 2;
            for (int it = tid; it < nk_all * npair && ready; it += DK_CT) {
                const int key = it % nk_all, r0 = (it / nk_all) * 2;
                const bool two = r0 + 1 < rep;
                const int32_t *kk;
                if (key < nk) { const unsigned sq = kseq + key / kps; kk = reinterpret_cast<const int32_t *>(slots + (size_t)(sq % DK_NS) * DK_SLOT) + (key % kps) * a.hd; }
                else kk = s_knew;
                const int32_t *qa = s_q + r0 * a.hd, *qb = s_q + (two ? r0 + 1 : r0) * a.hd;
                long long d0 = 0, d1 = 0;
                for (int j0 = 0; j0 < a.hd; j0 += 4) {
                    const int j = (j0 + 4 * key) & (a.hd - 1);     // every key starts at its own column: no bank conflicts on unpadded rows
                    const int4 k4 = *reinterpret_cast<const int4 *>(kk + j);
                    const int4 a4 = *reinterpret_cast<const int4 *>(qa + j), b4 = *reinterpret_cast<const int4 *>(qb + j);
                    d0 += (long long)a4.x * k4.x; d0 += (long long)a4.y * k4.y; d0 += (long long)a4.z * k4.z; d0 += (long long)a4.w * k4.w;
                    d1 += (long long)b4.x * k4.x; d1 += (long long)b4.y * k4.y; d1 += (long long)b4.z * k4.z; d1 += (long long)b4.w * k4.w;
                }
                const long long sc0 = ((d0 >> a.fa) * a.inv_sqrt) >> a.fa, sc1 = ((d1 >> a.fa) * a.inv_sqrt) >> a.fa;
                s_sc[key * rep + r0] = sc0;
                atomicMax(&sh->hmax[r0], sc0);
                if (two) { s_sc[key * rep + r0 + 1] = sc1; atomicMax(&sh->hmax[r0 + 1], sc1); }
            }
        }
        cbar();
        if (active && tid < rep && sh->hmax[tid] != INT64_MIN) atomicMax(hmax + kv * rep + tid, sh->hmax[tid]);
        if (tid == 0) for (int j = 0; j < kslots; j++) mb_arrive(&sh->empty[(kseq + j) % DK_NS]);     // key slots back to the producer
        seq += (unsigned)kslots;
        cbar();
        if (tid == 0) grid_arrive(a.bars, GB_MAX);

        share(sh->g.n_g, c, nc, i0, i1);
        lin_items<QT_Q4K>(a, sh, KIND_G, i0, i1, seq, half_h, planes, pstride);
        seq += (unsigned)(i1 - i0);
        cbar();
        if (tid == 0) { grid_arrive(a.bars, GB_GU); grid_wait(a.bars, GB_MAX, target, &sh->abort); }
        cbar();

        // ================================ P2: exponentials; down ================================
        if (active) {
            for (int it = tid; it < nk_all * rep; it += DK_CT) {
                const int r = it % rep;
                long long dlt = __ldcg(hmax + kv * rep + r) - s_sc[it];
                dlt = dlt < a.clip ? dlt : a.clip;
                const unsigned e = (unsigned)exp2_neg_fixed((dlt * a.log2e) >> a.fa, a.fa);
                s_e[it] = e;
                if (e) atomicAdd(&sh->z[r], (unsigned long long)e);
            }
        }
        cbar();
        if (active && tid < rep && sh->z[tid]) atomicAdd(Z + kv * rep + tid, sh->z[tid]);
        cbar();
        if (tid == 0) { grid_arrive(a.bars, GB_Z); grid_wait(a.bars, GB_GU, target, &sh->abort); }
        cbar();
        {
            int d0, d1;
            share(sh->g.n_d, c, nc, d0, d1);
            const int ipe = sh->g.ipe;
            unsigned dseq = seq;
            for (int i = d0; i < d1;) {                          // one routed expert at a time: its digit planes staged once
                const int s = i / ipe;
                const int iend = min(d1, (s + 1) * ipe);
                int nl = 1;
                for (int v = tid; v < 8 * (a.eff / 16); v += DK_CT) {
                    const int l = v / (a.eff / 16), o16 = v - l * (a.eff / 16);
                    const int4 w = __ldcg(reinterpret_cast<const int4 *>(a.gul + ((long long)s * 8 + l) * a.eff) + o16);
                    *reinterpret_cast<int4 *>(gup + l * gstride + o16 * 16) = w;
                    if ((w.x | w.y | w.z | w.w) != 0) nl = max(nl, l + 1);
                }
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, sft));
                if (tid == 0) sh->nl = 1;
                cbar();
                if (lane == 0) atomicMax(&sh->nl, nl);
                cbar();
                const bool half_g = sh->nl <= 4;
                if (ly.down_q == QT_Q6K) lin_items<QT_Q6K>(a, sh, KIND_D, i, iend, dseq, half_g, gup, gstride);
                else lin_items<QT_Q4K>(a, sh, KIND_D, i, iend, dseq, half_g, gup, gstride);
                dseq += (unsigned)(iend - i);
                i = iend;
                cbar();
            }
            seq = dseq;
        }

        // ================================ P3: probabilities x values ================================
        if (tid == 0) grid_wait(a.bars, GB_Z, target, &sh->abort);
        cbar();
        const unsigned vseq = seq;
        if (active) {
            for (int it = tid; it < nk_all * rep; it += DK_CT) {
                const unsigned long long z = __ldcg(Z + kv * rep + it % rep);
                s_e[it] = z ? (unsigned)(((unsigned long long)s_e[it] << a.fa) / z) : 0u;
            }
        }
        cbar();
        if (active) {
            bool ready = true;
            for (int j = 0; j < kslots; j++)
                ready = mb_wait(&sh->full[(vseq + j) % DK_NS], ((vseq + j) / DK_NS) & 1, &sh->abort) && ready;
            const int G = DK_CT / a.hd, grp = tid / a.hd, dcol = tid - grp * a.hd;
            if (grp < G && ready) {
                for (int r0 = grp * 2; r0 < rep; r0 += G * 2) {
                    const bool two = r0 + 1 < rep;
                    long long c0 = 0, c1 = 0;
                    for (int j = 0; j < kslots; j++) {
                        const int32_t *vs = reinterpret_cast<const int32_t *>(slots + (size_t)((vseq + j) % DK_NS) * DK_SLOT) + dcol;
                        const int n = min(kps, nk - j * kps);
                        const unsigned *pe = s_e + (size_t)j * kps * rep + r0;
                        for (int kk = 0; kk < n; kk++) {
                            const long long v = vs[kk * a.hd];
                            c0 += (long long)(int)pe[kk * rep] * v;
                            if (two) c1 += (long long)(int)pe[kk * rep + 1] * v;
                        }
                    }
                    if (owner) {
                        const long long v = s_vnew[dcol];
                        c0 += (long long)(int)s_e[nk * rep + r0] * v;
                        if (two) c1 += (long long)(int)s_e[nk * rep + r0 + 1] * v;
                    }
                    if (c0) atomicAdd(reinterpret_cast<unsigned long long *>(acc + (long long)(kv * rep + r0) * a.hd + dcol), (unsigned long long)c0);
                    if (two && c1) atomicAdd(reinterpret_cast<unsigned long long *>(acc + (long long)(kv * rep + r0 + 1) * a.hd + dcol), (unsigned long long)c1);
                }
            }
        }
        cbar();
        if (tid == 0) for (int j = 0; j < kslots; j++) mb_arrive(&sh->empty[(vseq + j) % DK_NS]);     // value slots back to the producer
        seq += (unsigned)kslots;
        if (tid == 0) { grid_arrive(a.bars, GB_ACC); grid_wait(a.bars, GB_ACC, target, &sh->abort); }
        cbar();

        // ================================ P4: O product ================================
        share(sh->g.to, c, nc, i0, i1);
        if (i1 > i0) {
            int nl = 1;
            bool over = false;
            const int kn = a.H * a.hd;
            for (int e0 = tid * 4; e0 < kn; e0 += DK_CT * 4) {
                uint32_t pw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const long long y = __ldcg(acc + e0 + e) >> a.fa;
                    bool ok;
                    const uint64_t dg = balanced_digits8(y, ok);
                    over |= !ok;
                    nl = max(nl, digits_used(dg));
#pragma unroll
                    for (int l = 0; l < 8; l++) pw[l] |= (uint32_t)((dg >> (8 * l)) & 0xFF) << (8 * e);
                }
#pragma unroll
                for (int l = 0; l < 8; l++) *reinterpret_cast<uint32_t *>(planes + l * pstride + e0) = pw[l];
            }
            if (over) atomicOr(a.flags, 1);
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) nl = max(nl, __shfl_xor_sync(0xffffffffu, nl, sft));
            if (tid == 0) sh->nl = 1;
            cbar();
            if (lane == 0) atomicMax(&sh->nl, nl);
            cbar();
            lin_items<QT_Q4K>(a, sh, KIND_O, i0, i1, seq, sh->nl <= 4, planes, pstride);
            seq += (unsigned)(i1 - i0) * (unsigned)sh->g.okn;
        }
        cbar();
        if (tid == 0) grid_arrive(a.bars, GB_X);
    }
    if (tid == 0 && sh->abort) atomicOr(a.flags, 8);
}

size_t decode_smem_bytes(int d, int H, int Hkv, int hd, int E, int eff) {
    const int pk = std::max(d, H * hd), rep = H / Hkv, maxkeys = DK_KSLOTS * (DK_SLOT / (hd * 4)) + 1;
    size_t n = (size_t)DK_NS * DK_SLOT + (size_t)DK_NS * 2 * 128 * 8 + (size_t)8 * (pk + DK_PAD) + (size_t)8 * (eff + DK_PAD);
    n += (size_t)((std::max(maxkeys * rep, E) + 1) & ~1) * 8 + (size_t)((maxkeys * rep + 3) & ~3) * 4 + (size_t)rep * hd * 4 + (size_t)2 * hd * 4;
    return n + 128;
}

// Largest number of history keys one launch can hold per KV head on `n_ctas` CTAs.
long long decode_key_capacity(int n_ctas, int Hkv, int hd) {
    return (long long)(n_ctas / Hkv) * DK_KSLOTS * (DK_SLOT / (hd * 4));
}

bool decode_shape_ok(int d, int H, int Hkv, int hd, int E, int k, int eff, int down_q) {
    if (d <= 0 || d % 256 || d > DK_CT * DK_EPT || eff <= 0 || eff % 256 || H <= 0 || Hkv <= 0 || H % Hkv) return false;
    const int rep = H / Hkv;
    if (rep > DK_MAXREP || hd < 32 || hd > 256 || (hd & (hd - 1)) || DK_CT % hd || (H * hd) % 256) return false;
    if (E <= 0 || E > 1024 || k <= 0 || k > E || k > DK_MAXK) return false;
    const int htb = down_q == QT_Q4K ? HTB_Q4K : HTB_Q6K;
    if (2 * (d / 256) * HTB_Q4K > DK_SLOT || 2 * (eff / 256) * htb > DK_SLOT) return false;     // a 16-row tile must fit a ring slot
    return decode_smem_bytes(d, H, Hkv, hd, E, eff) <= DK_SMEM_MAX;
}

cudaError_t launch_decode(const DecodeArgs &a, int n_ctas, cudaStream_t s) {
    const size_t smem = decode_smem_bytes(a.d, a.H, a.Hkv, a.hd, a.E, a.eff);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DK_SMEM_MAX);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaError_t e = cudaMemsetAsync(a.bars, 0, GB_COUNT * sizeof(unsigned), s);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_ctas); cfg.blockDim = dim3(DK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_kernel, a);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

int decode_max_ctas(int d, int H, int Hkv, int hd, int E, int eff) {
    int dev = 0, sms = 0, per_sm = 0, coop = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return 0;
    if (cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DK_SMEM_MAX) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_kernel, DK_THREADS, decode_smem_bytes(d, H, Hkv, hd, E, eff)) != cudaSuccess) {
        cudaGetLastError(); return 0;
    }
    return per_sm >= 1 ? sms : 0;
}

}  // namespace iie
