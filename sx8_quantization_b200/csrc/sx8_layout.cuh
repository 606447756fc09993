// sx8_layout.cuh -- the T16 device layout of an S-X8 v4.3 tensor.
//
// A byte/bit permutation of the 30-byte blocks, arranged so that (1) everything a
// CTA needs for a 16-column tile and a range of block rows kb is ONE contiguous
// range (one TMA bulk copy per pipeline stage), (2) a warp reads its operands with
// three conflict-free 32-bit shared-memory loads, and (3) the 6-bit levels come out
// as fp16 pairs with byte-parallel masks.
//
//   blob[(T*n_cb + kb) * 480 ...] : unit of tile T (columns 16T..16T+15), block row kb
//   lane L = 4g + t owns sub-block t (weights 8t..8t+7) of column A = 16T+g and of
//   column B = 16T+g+8.  a_i / b_i = 6-bit level of weight 8t+i of A / B:
//     W0 @ unit +   0 + 4L : bytes [a0,a2,a1,a3] << 2 | bits 1:0 of [b4,b6,b5,b7]
//     W1 @ unit + 128 + 4L : bytes [a4,a6,a5,a7] << 2 | bits 3:2 of [b4,b6,b5,b7]
//     W2 @ unit + 256 + 4L : bytes [b0,b2,b1,b3] << 2 | bits 5:4 of [b4,b6,b5,b7]
//     H0[g] @ unit + 384 + 4g : dmin(A) | dmax(A) << 16      (fp16 bits)
//     H1[g] @ unit + 416 + 4g : dmin(B) | dmax(B) << 16
//     H2[g] @ unit + 448 + 4g : c0(A) | c0(B)<<4 | config(A)<<8 | c1(A)<<16 | c1(B)<<20 | config(B)<<24
//                               (c0 / c1 = low / high nibble of the coeff byte)
//   Columns >= N are zero blocks.  Exactly 30 bytes per block.
#pragma once
#include <stdint.h>

namespace sx8 {

constexpr int T16_UNIT = 480;
constexpr int SX8_BLOCK_BYTES = 30;   // one interleaved block_sx8 record
constexpr int T16_LEV = 384;

__host__ __device__ inline long t16_tiles(long N) { return (N + 15) / 16; }
__host__ __device__ inline size_t t16_bytes(long N, long n_cb) { return (size_t)t16_tiles(N) * n_cb * T16_UNIT; }

// Everything of block (n, kb), sub-block t, read back from the blob (gather paths:
// embedding rows, full-tensor decode).
struct T16Sub {
    uint32_t lv[8];  // levels of weights 8t .. 8t+7
    uint32_t dmin, dmax, cfg, coeff;
};

__device__ __forceinline__ T16Sub t16_read(const uint8_t* __restrict__ blob, long n, long kb, int t, long n_cb) {
    long T = n >> 4;
    int r = (int)(n & 15), g = r & 7, isB = r >> 3;
    const uint32_t* u = reinterpret_cast<const uint32_t*>(blob + (T * n_cb + kb) * T16_UNIT);
    int L = g * 4 + t;
    uint32_t W0 = u[L], W1 = u[32 + L], W2 = u[64 + L];
    T16Sub s;
    if (!isB) {
        s.lv[0] = (W0 >> 2) & 63;  s.lv[1] = (W0 >> 18) & 63; s.lv[2] = (W0 >> 10) & 63; s.lv[3] = (W0 >> 26) & 63;
        s.lv[4] = (W1 >> 2) & 63;  s.lv[5] = (W1 >> 18) & 63; s.lv[6] = (W1 >> 10) & 63; s.lv[7] = (W1 >> 26) & 63;
    } else {
        s.lv[0] = (W2 >> 2) & 63;  s.lv[1] = (W2 >> 18) & 63; s.lv[2] = (W2 >> 10) & 63; s.lv[3] = (W2 >> 26) & 63;
        uint32_t V3 = ((W0 << 2) & 0x0C0C0C0Cu) | ((W1 << 4) & 0x30303030u) | ((W2 << 6) & 0xC0C0C0C0u);
        s.lv[4] = (V3 >> 2) & 63;  s.lv[5] = (V3 >> 18) & 63; s.lv[6] = (V3 >> 10) & 63; s.lv[7] = (V3 >> 26) & 63;
    }
    uint32_t h = u[96 + isB * 8 + g];
    uint32_t h2 = u[112 + g];
    s.dmin = h & 0xFFFFu;
    s.dmax = h >> 16;
    s.cfg = (h2 >> (8 + 16 * isB)) & 0xFFu;
    s.coeff = ((h2 >> (4 * isB)) & 0xFu) | (((h2 >> (16 + 4 * isB)) & 0xFu) << 4);
    return s;
}

}  // namespace sx8
