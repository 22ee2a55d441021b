// CPU replay of one warp of the IQ3_S matrix-vector kernel (test infrastructure).
//
// It runs the very decode helpers the CUDA kernel uses (iq3s_tile.h compiles for the host too) lane by lane, and
// models mma.sync.m16n8k32.s8 by the fragment layout the PTX ISA documents:
//   A (16x32, row): a0 = row g,   k 4q..4q+3;  a1 = row g+8, k 4q..4q+3;  a2 = row g, k 16+4q..;  a3 = row g+8, k 16+4q..
//   B (32x8,  col): b0 = k 4q..4q+3, col g;    b1 = k 16+4q..16+4q+3, col g
//   C (16x8):       c0, c1 = row g, cols 2q, 2q+1;   c2, c3 = row g+8, cols 2q, 2q+1
// so that the tile layout, the 9-bit field extraction, the sign masks and the activation cell layout can be checked
// against the oracle without a GPU.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "iq3s_grid.h"
#include "iq3s_tile.h"

using namespace fnxb;

static const uint32_t kGrid[512] = {FNX_IQ3S_GRID_VALUES};

template <int I>
static uint32_t dec(const uint32_t (&S)[5], const uint32_t (&G)[2], int lane) {
    const uint32_t off = tile_field<I>(S) | (uint32_t) (lane * 4);
    const uint32_t mag = kGrid[off >> 7];   // the replicated table holds entry (off >> 7) at every lane slot
    return tile_apply_sign(mag, tile_sign_mask<I>(G));
}

template <int SB>
static void sub_block(const uint32_t (&S0)[5], const uint32_t (&G0)[2], const uint32_t (&S1)[5], const uint32_t (&G1)[2], int lane,
                      uint32_t (&a)[4]) {
    a[0] = dec<2 * SB>(S0, G0, lane);
    a[2] = dec<2 * SB + 1>(S0, G0, lane);
    a[1] = dec<2 * SB>(S1, G1, lane);
    a[3] = dec<2 * SB + 1>(S1, G1, lane);
}

static uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static float h2f(uint16_t h) {
    const uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 31u, m = h & 1023u;
    float f = e == 0 ? ldexpf((float) m, -24) : ldexpf((float) (m + 1024u), (int) e - 25);
    return s ? -f : f;
}

// y[t][r] for t < T <= 4: one token group, two int8 levels in the 8 MMA columns
extern "C" void sim_mmv(const uint8_t* ggml, int rows, int K, const float* x, int T, float* y) {
    const int KB = K / 256;
    std::vector<uint8_t> tiles((size_t) rows * KB * IQ3S_BLOCK_BYTES);
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < KB; ++b)
            tile_put_block(tiles.data() + ((size_t) (r / 16) * KB + b) * TILE_BYTES, r % 16, ggml + ((size_t) r * KB + b) * IQ3S_BLOCK_BYTES);
    // activation cells [sbG][n][q] (8 int8 each) and scales [blk][8]
    std::vector<int8_t> xq((size_t) (K / 32) * 32 * 8, 0);
    std::vector<float> xs((size_t) KB * 8, 0.f);
    for (int t = 0; t < T; ++t)
        for (int b = 0; b < KB; ++b) {
            const float* xr = x + (size_t) t * K + b * 256;
            float am = 0.f;
            for (int i = 0; i < 256; ++i) am = fmaxf(am, fabsf(xr[i]));
            const float d = am / 127.0f, inv = am > 0.f ? 127.0f / am : 0.f, inv2 = inv * 256.0f;
            xs[b * 8 + t] = d;
            xs[b * 8 + t + 4] = d * (1.0f / 256.0f);
            for (int i = 0; i < 256; ++i) {
                int a1 = (int) rintf(xr[i] * inv);
                a1 = a1 > 127 ? 127 : a1 < -127 ? -127 : a1;
                int a2 = (int) rintf((xr[i] - (float) a1 * d) * inv2);
                a2 = a2 > 127 ? 127 : a2 < -127 ? -127 : a2;
                const int sbG = b * 8 + i / 32, q = (i % 32) / 8, j = i % 8;
                xq[(((size_t) sbG * 8 + t) * 4 + q) * 8 + j] = (int8_t) a1;
                xq[(((size_t) sbG * 8 + t + 4) * 4 + q) * 8 + j] = (int8_t) a2;
            }
        }
    for (int rt = 0; rt < rows / 16; ++rt) {
        float out[16][8];
        memset(out, 0, sizeof out);
        for (int b = 0; b < KB; ++b) {
            const uint8_t* tile = tiles.data() + ((size_t) rt * KB + b) * TILE_BYTES;
            for (int lane = 0; lane < 32; ++lane) {
                const int g = lane >> 2, q = lane & 3;
                uint32_t S0[5], S1[5], G0[2], G1[2];
                for (int j = 0; j < 4; ++j) {
                    S0[j] = rd32(tile + TILE_IDX + lane * 16 + 4 * j);
                    S1[j] = rd32(tile + TILE_IDX + 512 + lane * 16 + 4 * j);
                }
                S0[4] = rd16(tile + TILE_TAIL + lane * 2);
                S1[4] = rd16(tile + TILE_TAIL + 64 + lane * 2);
                for (int j = 0; j < 2; ++j) {
                    G0[j] = rd32(tile + TILE_SGN + lane * 8 + 4 * j);
                    G1[j] = rd32(tile + TILE_SGN + 256 + lane * 8 + 4 * j);
                }
                const uint32_t sc0 = rd32(tile + TILE_SCL + g * 4), sc1 = rd32(tile + TILE_SCL + (g + 8) * 4);
                const float d0 = h2f(rd16(tile + TILE_D + g * 2)), d1 = h2f(rd16(tile + TILE_D + (g + 8) * 2));
                int accI[4] = {0, 0, 0, 0};
                uint32_t a[8][4];
                sub_block<0>(S0, G0, S1, G1, lane, a[0]); sub_block<1>(S0, G0, S1, G1, lane, a[1]);
                sub_block<2>(S0, G0, S1, G1, lane, a[2]); sub_block<3>(S0, G0, S1, G1, lane, a[3]);
                sub_block<4>(S0, G0, S1, G1, lane, a[4]); sub_block<5>(S0, G0, S1, G1, lane, a[5]);
                sub_block<6>(S0, G0, S1, G1, lane, a[6]); sub_block<7>(S0, G0, S1, G1, lane, a[7]);
                // This lane's A registers cover MMA k = 4q..4q+3 (a0/a1) and 16+4q.. (a2/a3) of rows g, g+8.  The MMA
                // sums over all four threads of the row group; model it by letting this lane add ITS k-slice of the
                // products to every column's accumulator (the C layout then just says who ends up holding them).
                for (int sb = 0; sb < 8; ++sb) {
                    const int w0 = 1 + 2 * (int) ((sc0 >> (4 * sb)) & 15u), w1 = 1 + 2 * (int) ((sc1 >> (4 * sb)) & 15u);
                    for (int n = 0; n < 8; ++n) {
                        // B fragment of the thread (n, q): the cell [sbG][n][q]: b0 = bytes 0..3, b1 = bytes 4..7
                        const int8_t* cell = &xq[(((size_t) (b * 8 + sb) * 8 + n) * 4 + q) * 8];
                        int c0 = 0, c1 = 0;
                        for (int j = 0; j < 4; ++j) {
                            c0 += (int) (int8_t) (a[sb][0] >> (8 * j)) * cell[j] + (int) (int8_t) (a[sb][2] >> (8 * j)) * cell[4 + j];
                            c1 += (int) (int8_t) (a[sb][1] >> (8 * j)) * cell[j] + (int) (int8_t) (a[sb][3] >> (8 * j)) * cell[4 + j];
                        }
                        out[g][n] += d0 * xs[b * 8 + n] * (float) (w0 * c0);
                        out[g + 8][n] += d1 * xs[b * 8 + n] * (float) (w1 * c1);
                    }
                }
                (void) accI;
            }
        }
        for (int r = 0; r < 16; ++r)
            for (int t = 0; t < T; ++t) y[(size_t) t * rows + rt * 16 + r] = out[r][t] + out[r][t + 4];
    }
}

extern "C" void sim_roundtrip(const uint8_t* ggml, int rows, int K, uint8_t* back) {
    const int KB = K / 256;
    std::vector<uint8_t> tiles((size_t) rows * KB * IQ3S_BLOCK_BYTES);
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < KB; ++b)
            tile_put_block(tiles.data() + ((size_t) (r / 16) * KB + b) * TILE_BYTES, r % 16, ggml + ((size_t) r * KB + b) * IQ3S_BLOCK_BYTES);
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < KB; ++b)
            tile_get_block(tiles.data() + ((size_t) (r / 16) * KB + b) * TILE_BYTES, r % 16, back + ((size_t) r * KB + b) * IQ3S_BLOCK_BYTES);
}
