// Device-resident weight layout ("half-tile" repack) for Q4_K / Q6_K tensors.
//
// The registry owns its device copy of every weight, so it stores the raw GGUF blocks
// (north-mini-code/src/nmc/qk_codec.py:16-18: Q4_K = d,dmin,scales[12],qs[128]; Q6_K =
// ql[128],qh[64],scales[16],d) re-ordered so that a warp streams them with 128-bit, fully coalesced
// loads that land directly in tensor-core A-fragment order.  No bit of a block changes; a tensor
// occupies exactly out_f_padded * n_blocks * {144|210} bytes (rows padded to a multiple of 8 with
// zero blocks, which decode to zero weights).
//
// Unit: one "half-tile block" = 8 consecutive output rows x one 256-column super-block.
// Tensor = [half_tile][block][bytes].  Inside a unit, lane = 4*row + t (row 0..7, t 0..3).
//
// Q4_K unit (1152 B):
//   [   0,1024)  nibbles: [pair p=0..1][lane][16 B] = row's qs[64p + 8t .. +7] then qs[64p + 32 + 8t .. +7]
//                (group G = 2p + {0,1}; low nibbles are sub-block 2G, high nibbles sub-block 2G+1)
//   [1024,1152)  per row 16 B: d, dmin, scales[12]   (the block's first 16 raw bytes)
// Q6_K unit (1680 B):
//   [   0,1024)  low nibbles: [half h=0..1][lane][16 B] = for u=0,1: ql[64h + 16u + 4t .. +3], ql[64h + 32 + 16u + 4t .. +3]
//   [1024,1536)  high bits:   [lane][16 B] = for (h,u): qh[32h + 16u + 4t .. +3]
//   [1536,1664)  per row 16 B: int8 scales[16]
//   [1664,1680)  per row 2 B: d
#pragma once
#include "common.cuh"

namespace iie {

// Offset inside a Q4_K unit of raw byte `i` (0..143) of row `r` (0..7).
__host__ __device__ inline int q4k_unit_offset(int r, int i) {
    if (i < 16) return 1024 + r * 16 + i;
    const int q = i - 16, G = q >> 5, w = q & 31, t = w >> 3, k = w & 7;
    return (G >> 1) * 512 + (r * 4 + t) * 16 + (G & 1) * 8 + k;
}

// Offset inside a Q6_K unit of raw byte `i` (0..209) of row `r` (0..7).
__host__ __device__ inline int q6k_unit_offset(int r, int i) {
    if (i < 128) {                       // ql
        const int h = i >> 6, rr = i & 63, isB = rr >> 5, l = rr & 31, u = l >> 4, t = (l & 15) >> 2, k = l & 3;
        return h * 512 + (r * 4 + t) * 16 + u * 8 + isB * 4 + k;
    }
    if (i < 192) {                       // qh
        const int q = i - 128, h = q >> 5, l = q & 31, u = l >> 4, t = (l & 15) >> 2, k = l & 3;
        return 1024 + (r * 4 + t) * 16 + (h * 2 + u) * 4 + k;
    }
    if (i < 208) return 1536 + r * 16 + (i - 192);
    return 1664 + r * 2 + (i - 208);
}

// Byte `i` of the raw block (row, block) read back from a repacked tensor.
__device__ inline uint8_t repacked_byte(const uint8_t *w, int qtype, long long n_blocks, long long row, long long blk, int i) {
    const long long unit = (row >> 3) * n_blocks + blk;
    const int r = (int)(row & 7);
    return qtype == QT_Q4K ? w[unit * HTB_Q4K + q4k_unit_offset(r, i)] : w[unit * HTB_Q6K + q6k_unit_offset(r, i)];
}

}  // namespace iie
