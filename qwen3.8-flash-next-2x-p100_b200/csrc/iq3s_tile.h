// IQ3_S on the device: the 16-row tile layout and its decode steps.
//
// The interchange format stays GGML's block_iq3_s (110 bytes per 256 weights: d f16 @0, qs[64] @2, qh[8] @66,
// signs[32] @74, scales[4] @106; the reference reads it at engine/src/moe_mma_iq.cuh:146-185 and
// engine/src/tensor_convert.hpp:295-322).  At load time every matrix is re-tiled, bit for bit (a permutation of
// the same bits, still 110 bytes per 256 weights), into tiles of 16 rows x 256 columns laid out for one warp
// that feeds mma.sync.m16n8k32.s8 with the weights as the A operand:
//
//   lane = 4 g + q  (g = 0..7 the fragment row, q = 0..3 the thread in its group) owns, of rows g and g + 8,
//   the 8 weights 8 q .. 8 q + 7 of every 32-weight sub-block: two codebook indices and 8 sign bits per
//   sub-block, 16 indices and 64 sign bits per row and 256-column block.
//
//   offset    bytes  content
//   0         1024   index streams: [half h][g][q] 16 bytes = bits 0..127 of the lane's 144-bit stream for row
//                    8 h + g: index i = 2 sb + e (sub-block sb, e = 0: weights 8q..8q+3, e = 1: 8q+4..8q+7) is
//                    the 9-bit field at bit 9 i  (qs byte | qh bit << 8)
//   1024       512   sign words: [h][g][q] two u32: word i >> 3, bit 8 j + (i & 7) = sign of weight j of index i
//   1536       128   stream tails: [h][g][q] u16 = bits 128..143 of the index stream
//   1664        64   scales: [row] u32, nibble sb = the sub-block's 4-bit scale s (weight scale d (1 + 2 s))
//   1728        32   d: [row] f16
//
// A matrix of R rows x K columns is the sequence of tiles [R / 16][K / 256], 1760 bytes each, so any run of tiles
// is one contiguous, 16-byte aligned span that a bulk async copy can stage into shared memory.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define FNX_HD __host__ __device__ __forceinline__
#else
#define FNX_HD inline
#endif

namespace fnxb {

constexpr int IQ3S_BLOCK_BYTES = 110;
constexpr int TILE_ROWS = 16;
constexpr int TILE_BYTES = 1760;
constexpr int TILE_IDX = 0, TILE_SGN = 1024, TILE_TAIL = 1536, TILE_SCL = 1664, TILE_D = 1728;

// bytes of an R x K matrix (either layout)
FNX_HD size_t iq3s_bytes(size_t rows, size_t cols) { return rows * (cols / 256) * IQ3S_BLOCK_BYTES; }

// Writes row r (0..15) of a tile from its GGML block.  `tile` must be zeroed beforehand only in its index-stream,
// sign and tail planes' parts for this row (this function overwrites them fully).
FNX_HD void tile_put_block(uint8_t* tile, int r, const uint8_t* blk) {
    const uint8_t *qs = blk + 2, *qh = blk + 66, *signs = blk + 74, *scales = blk + 106;
    const int lane0 = r * 4;   // (h * 8 + g) * 4
    for (int q = 0; q < 4; ++q) {
        uint32_t w[6] = {0, 0, 0, 0, 0, 0};
        uint32_t sg[2] = {0, 0};
        for (int sb = 0; sb < 8; ++sb)
            for (int e = 0; e < 2; ++e) {
                const int i = 2 * sb + e, k = 2 * q + e;
                const uint32_t idx = (uint32_t) qs[8 * sb + k] | ((((uint32_t) qh[sb] >> k) & 1u) << 8);
                const int o = 9 * i, j = o >> 5, s = o & 31;
                w[j] |= idx << s;
                if (s > 23) w[j + 1] |= idx >> (32 - s);
                const uint32_t sbyte = signs[4 * sb + q];
                for (int jj = 0; jj < 4; ++jj) sg[i >> 3] |= ((sbyte >> (4 * e + jj)) & 1u) << (8 * jj + (i & 7));
            }
        uint8_t* pi = tile + TILE_IDX + (lane0 + q) * 16;
        for (int j = 0; j < 4; ++j) {
            pi[4 * j] = (uint8_t) w[j];
            pi[4 * j + 1] = (uint8_t) (w[j] >> 8);
            pi[4 * j + 2] = (uint8_t) (w[j] >> 16);
            pi[4 * j + 3] = (uint8_t) (w[j] >> 24);
        }
        uint8_t* pt = tile + TILE_TAIL + (lane0 + q) * 2;
        pt[0] = (uint8_t) w[4];
        pt[1] = (uint8_t) (w[4] >> 8);
        uint8_t* ps = tile + TILE_SGN + (lane0 + q) * 8;
        for (int j = 0; j < 2; ++j) {
            ps[4 * j] = (uint8_t) sg[j];
            ps[4 * j + 1] = (uint8_t) (sg[j] >> 8);
            ps[4 * j + 2] = (uint8_t) (sg[j] >> 16);
            ps[4 * j + 3] = (uint8_t) (sg[j] >> 24);
        }
    }
    for (int j = 0; j < 4; ++j) tile[TILE_SCL + r * 4 + j] = scales[j];
    tile[TILE_D + r * 2] = blk[0];
    tile[TILE_D + r * 2 + 1] = blk[1];
}

// The inverse: row r of a tile back to its GGML block (used to show the re-tiling loses nothing).
FNX_HD void tile_get_block(const uint8_t* tile, int r, uint8_t* blk) {
    for (int i = 0; i < IQ3S_BLOCK_BYTES; ++i) blk[i] = 0;
    uint8_t *qs = blk + 2, *qh = blk + 66, *signs = blk + 74, *scales = blk + 106;
    const int lane0 = r * 4;
    for (int q = 0; q < 4; ++q) {
        uint32_t w[6] = {0, 0, 0, 0, 0, 0}, sg[2];
        const uint8_t* pi = tile + TILE_IDX + (lane0 + q) * 16;
        for (int j = 0; j < 4; ++j)
            w[j] = (uint32_t) pi[4 * j] | ((uint32_t) pi[4 * j + 1] << 8) | ((uint32_t) pi[4 * j + 2] << 16) | ((uint32_t) pi[4 * j + 3] << 24);
        const uint8_t* pt = tile + TILE_TAIL + (lane0 + q) * 2;
        w[4] = (uint32_t) pt[0] | ((uint32_t) pt[1] << 8);
        const uint8_t* ps = tile + TILE_SGN + (lane0 + q) * 8;
        for (int j = 0; j < 2; ++j)
            sg[j] = (uint32_t) ps[4 * j] | ((uint32_t) ps[4 * j + 1] << 8) | ((uint32_t) ps[4 * j + 2] << 16) | ((uint32_t) ps[4 * j + 3] << 24);
        for (int sb = 0; sb < 8; ++sb)
            for (int e = 0; e < 2; ++e) {
                const int i = 2 * sb + e, k = 2 * q + e;
                const int o = 9 * i, j = o >> 5, s = o & 31;
                uint32_t idx = w[j] >> s;
                if (s > 23) idx |= w[j + 1] << (32 - s);
                idx &= 511u;
                qs[8 * sb + k] = (uint8_t) (idx & 255u);
                qh[sb] |= (uint8_t) (((idx >> 8) & 1u) << k);
                for (int jj = 0; jj < 4; ++jj)
                    signs[4 * sb + q] |= (uint8_t) (((sg[i >> 3] >> (8 * jj + (i & 7))) & 1u) << (4 * e + jj));
            }
    }
    for (int j = 0; j < 4; ++j) scales[j] = tile[TILE_SCL + r * 4 + j];
    blk[0] = tile[TILE_D + r * 2];
    blk[1] = tile[TILE_D + r * 2 + 1];
}

// ---- the decode steps of one lane, written so that the host can run them too (the tests replay a whole warp on
// the CPU against the oracle) ----

// byte offset of index i's codebook entry in the replicated table: (idx << 7), i.e. the 9-bit field moved to bits
// 7..15.  S[0..3] = the 16-byte stream, S[4] = its 16-bit tail.
// On the device the shifts are written as multiplies (x >> s == umulhi(x, 2^(32-s)), x << s == x * 2^s) by powers of
// two read from constant memory, so that they stay multiplies: integer multiply-add runs on the FMA pipes, which
// leaves the narrower integer-logic pipe to the masks and byte permutes (the decode is bound by that pipe).
#if defined(__CUDACC__)
__constant__ static uint32_t g_pow2[33] = {1u << 0,  1u << 1,  1u << 2,  1u << 3,  1u << 4,  1u << 5,  1u << 6,  1u << 7,  1u << 8,  1u << 9,  1u << 10,
                                           1u << 11, 1u << 12, 1u << 13, 1u << 14, 1u << 15, 1u << 16, 1u << 17, 1u << 18, 1u << 19, 1u << 20, 1u << 21,
                                           1u << 22, 1u << 23, 1u << 24, 1u << 25, 1u << 26, 1u << 27, 1u << 28, 1u << 29, 1u << 30, 1u << 31, 0u};
#endif
template <int I>
FNX_HD uint32_t tile_field(const uint32_t (&S)[5]) {
    constexpr int o = 9 * I, j = o >> 5, r = o & 31;
    uint32_t v;
    if constexpr (r >= 7 && r + 9 <= 32) {
#if defined(__CUDA_ARCH__)
        if constexpr (r == 7) v = S[j];
        else v = __umulhi(S[j], g_pow2[32 - (r - 7)]);
#else
        v = S[j] >> (r - 7);
#endif
    } else if constexpr (r >= 7) {
#if defined(__CUDA_ARCH__)
        v = __funnelshift_r(S[j], S[j + 1], r - 7);
#else
        v = (uint32_t) ((((uint64_t) S[j + 1] << 32) | S[j]) >> (r - 7));
#endif
    } else {
#if defined(__CUDA_ARCH__)
        v = S[j] * g_pow2[7 - r];
#else
        v = S[j] << (7 - r);
#endif
    }
    return v & 0xFF80u;
}

// byte mask (0xFF where the weight is negative) of index i's four weights from the lane's sign words
template <int I>
FNX_HD uint32_t tile_sign_mask(const uint32_t (&G)[2]) {
#if defined(__CUDA_ARCH__)
    uint32_t p = G[I >> 3], m;
    if constexpr ((I & 7) != 7) p = G[I >> 3] * g_pow2[7 - (I & 7)];
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(p), "r"(0u), "r"(0xBA98u));
    return m;
#else
    const uint32_t p = G[I >> 3] << (7 - (I & 7));
    uint32_t m = 0;
    for (int b = 0; b < 4; ++b)
        if ((p >> (8 * b + 7)) & 1u) m |= 0xFFu << (8 * b);
    return m;
#endif
}

// four codebook magnitudes (odd, 1..15, one per byte) with the signs applied as two's-complement int8: for an odd
// byte g, -g == g ^ 0xFE
FNX_HD uint32_t tile_apply_sign(uint32_t mag, uint32_t mask) { return mag ^ (mask & 0xFEFEFEFEu); }

}  // namespace fnxb
