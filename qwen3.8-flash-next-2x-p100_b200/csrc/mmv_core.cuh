// The inner pieces of the IQ3_S matrix x few-rows product, shared by the persistent step kernel: codebook table,
// one 16 x 256 tile against quantised activation cells, and the two-level int8 quantiser of activation rows.
//
// Activation image (in shared or global memory, same layout): rows in groups of four,
//   cells  uint2 [group][sub-block sbG = k / 32][column n = (row & 3) + 4 * level][q = (k % 32) / 8]   8 int8 each
//   scales float [group][block = k / 256][column n]                                                  d, d / 256
// so that the 8 columns of one mma.sync.m16n8k32.s8 hold both levels of up to four rows.
#pragma once

#include <cuda_fp16.h>

#include "fnx_common.cuh"
#include "iq3s_grid.h"
#include "iq3s_tile.h"

namespace fnxb {

__device__ static const uint32_t g_grid_core[512] = {FNX_IQ3S_GRID_VALUES};

constexpr int CORE_TABLE_BYTES = 512 * 128;
constexpr int CORE_ITEMS = 16;                              // (tile, block) items of one step
constexpr int CORE_STEP_BYTES = CORE_ITEMS * TILE_BYTES;    // 28,160

__device__ __forceinline__ size_t img_cells(int rows, int K) { return (size_t) ((rows + 3) / 4) * (K / 32) * 32; }   // uint2 cells
__device__ __forceinline__ size_t img_scales(int rows, int K) { return (size_t) ((rows + 3) / 4) * (K / 256) * 8; }  // floats
__host__ __device__ __forceinline__ size_t img_bytes(int rows, int K) {
    return (size_t) ((rows + 3) / 4) * ((size_t) (K / 32) * 32 * 8 + (size_t) (K / 256) * 8 * 4);
}

// the codebook, one copy per bank: entry e at byte e * 128 + 4 * lane
__device__ __forceinline__ void core_fill_table(uint8_t* table, int tid, int nthreads) {
    for (int e = tid; e < 512; e += nthreads) {
        const uint32_t v = g_grid_core[e];
        uint4* d = reinterpret_cast<uint4*>(table + e * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = make_uint4(v, v, v, v);
    }
}

__device__ __forceinline__ void core_mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// four s32 -> four saturated s8 in one word (byte 0 = a)
__device__ __forceinline__ uint32_t core_pack_s8x4(int a, int b, int c, int d) {
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}

template <int I>
__device__ __forceinline__ uint32_t core_decode(const uint32_t (&S)[5], const uint32_t (&G)[2], const uint8_t* table, uint32_t lane4) {
    const uint32_t off = tile_field<I>(S) | lane4;
    const uint32_t mag = *reinterpret_cast<const uint32_t*>(table + off);
    return tile_apply_sign(mag, tile_sign_mask<I>(G));
}

// What one lane reads of the activations: for each row group, its B cells (column = lane / 4) and the scales of its
// two C columns (2 q, 2 q + 1); null = an empty column.
template <int NG>
struct LaneX {
    const uint2* b[NG];
    const float* s0[NG];
    const float* s1[NG];
};

// lane pointers for a dense product over rows [0, T): group ng holds rows 4 ng .. 4 ng + 3
template <int NG>
__device__ __forceinline__ LaneX<NG> lane_x_dense(const uint2* xq, const float* xs, int K, int T, int lane) {
    LaneX<NG> lx;
    const int g = lane >> 2, q = lane & 3, KB = K / 256;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        lx.b[ng] = 4 * ng + (g & 3) < T ? xq + (size_t) ng * (K / 32) * 32 + lane : nullptr;
        const int c0 = 2 * q, c1 = 2 * q + 1;
        lx.s0[ng] = 4 * ng + (c0 & 3) < T ? xs + (size_t) ng * KB * 8 + c0 : nullptr;
        lx.s1[ng] = 4 * ng + (c1 & 3) < T ? xs + (size_t) ng * KB * 8 + c1 : nullptr;
    }
    return lx;
}

// lane pointers for one expert job over the image of all window rows: column n < 4 = level 1 of row y[n], n >= 4 = level 2
__device__ __forceinline__ LaneX<1> lane_x_job(const uint2* xq, const float* xs, int K, const int* y, int ntok, int lane) {
    LaneX<1> lx;
    const int g = lane >> 2, q = lane & 3, KB = K / 256;
    lx.b[0] = nullptr;
    if ((g & 3) < ntok) {
        const int row = y[g & 3];
        lx.b[0] = xq + ((size_t) (row >> 2) * (K / 32) * 8 + (row & 3) + 4 * (g >> 2)) * 4 + q;
    }
    const int c0 = 2 * q, c1 = 2 * q + 1;
    lx.s0[0] = lx.s1[0] = nullptr;
    if ((c0 & 3) < ntok) {
        const int row = y[c0 & 3];
        lx.s0[0] = xs + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c0 >> 2);
    }
    if ((c1 & 3) < ntok) {
        const int row = y[c1 & 3];
        lx.s1[0] = xs + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c1 >> 2);
    }
    return lx;
}

template <int NG, int SB>
__device__ __forceinline__ void core_sub_block(const uint32_t (&S0)[5], const uint32_t (&G0)[2], const uint32_t (&S1)[5], const uint32_t (&G1)[2],
                                               uint32_t sc0, uint32_t sc1, const uint8_t* table, uint32_t lane4, const LaneX<NG>& lx, int blk,
                                               int (&accI)[NG][4]) {
    const uint32_t a0 = core_decode<2 * SB>(S0, G0, table, lane4);
    const uint32_t a2 = core_decode<2 * SB + 1>(S0, G0, table, lane4);
    const uint32_t a1 = core_decode<2 * SB>(S1, G1, table, lane4);
    const uint32_t a3 = core_decode<2 * SB + 1>(S1, G1, table, lane4);
    // 1 + 2 s from the nibble: ((word >> (4 SB - 1)) & 30) | 1
    const int w0 = (int) ((SB ? (sc0 >> (4 * SB - 1)) : (sc0 << 1)) & 30u) | 1, w1 = (int) ((SB ? (sc1 >> (4 * SB - 1)) : (sc1 << 1)) & 30u) | 1;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        uint2 b = make_uint2(0u, 0u);
        if (lx.b[ng]) b = lx.b[ng][(size_t) (blk * 8 + SB) * 32];
        int c[4];
        core_mma_s8(c, a0, a1, a2, a3, b.x, b.y);
        accI[ng][0] += w0 * c[0];
        accI[ng][1] += w0 * c[1];
        accI[ng][2] += w1 * c[2];
        accI[ng][3] += w1 * c[3];
    }
}

// One item: tile (16 rows x 256 columns, block `blk` of its rows) against the lane's activation cells; adds into
// acc[ng][0..3] = (row g, col 2q), (row g, col 2q+1), (row g+8, col 2q), (row g+8, col 2q+1).
template <int NG>
__device__ __forceinline__ void core_item(const uint8_t* tile, const uint8_t* table, const LaneX<NG>& lx, int blk, int lane, float (&acc)[NG][4]) {
    const int g = lane >> 2;
    const uint32_t lane4 = (uint32_t) lane * 4u;
    const uint4 i0 = *reinterpret_cast<const uint4*>(tile + TILE_IDX + lane * 16);
    const uint4 i1 = *reinterpret_cast<const uint4*>(tile + TILE_IDX + 512 + lane * 16);
    const uint2 s0 = *reinterpret_cast<const uint2*>(tile + TILE_SGN + lane * 8);
    const uint2 s1 = *reinterpret_cast<const uint2*>(tile + TILE_SGN + 256 + lane * 8);
    const uint32_t t0 = *reinterpret_cast<const uint16_t*>(tile + TILE_TAIL + lane * 2);
    const uint32_t t1 = *reinterpret_cast<const uint16_t*>(tile + TILE_TAIL + 64 + lane * 2);
    const uint32_t sc0 = *reinterpret_cast<const uint32_t*>(tile + TILE_SCL + g * 4);
    const uint32_t sc1 = *reinterpret_cast<const uint32_t*>(tile + TILE_SCL + (g + 8) * 4);
    const float d0 = __half2float(*reinterpret_cast<const __half*>(tile + TILE_D + g * 2));
    const float d1 = __half2float(*reinterpret_cast<const __half*>(tile + TILE_D + (g + 8) * 2));
    const uint32_t S0[5] = {i0.x, i0.y, i0.z, i0.w, t0}, S1[5] = {i1.x, i1.y, i1.z, i1.w, t1};
    const uint32_t G0[2] = {s0.x, s0.y}, G1[2] = {s1.x, s1.y};
    int accI[NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int i = 0; i < 4; ++i) accI[ng][i] = 0;
    core_sub_block<NG, 0>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 1>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 2>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 3>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 4>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 5>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 6>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
    core_sub_block<NG, 7>(S0, G0, S1, G1, sc0, sc1, table, lane4, lx, blk, accI);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        const float x0 = lx.s0[ng] ? lx.s0[ng][blk * 8] : 0.f, x1 = lx.s1[ng] ? lx.s1[ng][blk * 8] : 0.f;
        acc[ng][0] += d0 * x0 * (float) accI[ng][0];
        acc[ng][1] += d0 * x1 * (float) accI[ng][1];
        acc[ng][2] += d1 * x0 * (float) accI[ng][2];
        acc[ng][3] += d1 * x1 * (float) accI[ng][3];
    }
}

// Quantises 8 consecutive values of one lane (a cell) given the block's maximum over the warp; returns the cells
__device__ __forceinline__ void core_quant_cell(const float (&x8)[8], float am, uint2& c1, uint2& c2, float& d) {
    d = am / 127.0f;
    const float inv = am > 0.f ? 127.0f / am : 0.f, inv2 = inv * 256.0f;
    int a8[8], b8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a8[i] = __float2int_rn(x8[i] * inv);
        b8[i] = __float2int_rn((x8[i] - (float) a8[i] * d) * inv2);
    }
    c1 = make_uint2(core_pack_s8x4(a8[0], a8[1], a8[2], a8[3]), core_pack_s8x4(a8[4], a8[5], a8[6], a8[7]));
    c2 = make_uint2(core_pack_s8x4(b8[0], b8[1], b8[2], b8[3]), core_pack_s8x4(b8[4], b8[5], b8[6], b8[7]));
}

}  // namespace fnxb
