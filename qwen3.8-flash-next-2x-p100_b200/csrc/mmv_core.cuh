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
    // a warp writes 32 entries: each store instruction covers 4 whole entries (512 contiguous bytes: no bank conflicts)
    const int warp = tid >> 5, lane = tid & 31, nwarp = nthreads >> 5;
    for (int e0 = warp * 32; e0 < 512; e0 += nwarp * 32) {
        const uint32_t mine = g_grid_core[e0 + lane];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t v = __shfl_sync(0xffffffffu, mine, 4 * i + (lane >> 3));
            *reinterpret_cast<uint4*>(table + (e0 + 4 * i) * 128 + lane * 16) = make_uint4(v, v, v, v);
        }
    }
}

__device__ __forceinline__ void core_mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
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

// shared-memory loads by 32-bit shared address plus a compile-time offset that rides in the instruction: no 64-bit
// generic pointer arithmetic and no address adds in the decode loop
template <int OFF = 0>
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF = 0>
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint16_t v;
    asm("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF = 0>
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF = 0>
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF = 0>
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
    return v;
}

template <int I>
__device__ __forceinline__ uint32_t core_decode(const uint32_t (&S)[5], const uint32_t (&G)[2], uint32_t table_s, uint32_t lane4) {
    // (field & 0xFF80) | 4 lane: one logic op; the table's (uniform) shared address rides in the load's address
    const uint32_t off = tile_field<I>(S) | lane4;
    const uint32_t mag = lds_u32(table_s + off);
    return tile_apply_sign(mag, tile_sign_mask<I>(G));
}

// What one lane reads of the activations: for each row group, its B cells (column = lane / 4) and the scales of its
// two C columns (2 q, 2 q + 1); null = an empty column.
template <int NG>
struct LaneX {
    uint32_t b[NG];     // shared addresses; 0 = an empty column
    uint32_t s0[NG];
    uint32_t s1[NG];
    float r0[NG], r1[NG];   // factors of the two C columns' rows (1 / rms of a normed row, else 1)
};

// lane pointers for a dense product over rows [0, T): group ng holds rows 4 ng .. 4 ng + 3
// (T >= 4 NG: every column gets its address; rows that hold nothing must then be zero cells with zero scales)
template <int NG>
__device__ __forceinline__ LaneX<NG> lane_x_dense(const uint2* xq, const float* xs, int K, int T, int lane) {
    LaneX<NG> lx;
    const int g = lane >> 2, q = lane & 3, KB = K / 256;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        lx.b[ng] = 4 * ng + (g & 3) < T ? smem_u32(xq + (size_t) ng * (K / 32) * 32 + lane) : 0u;
        const int c0 = 2 * q, c1 = 2 * q + 1;
        lx.s0[ng] = 4 * ng + (c0 & 3) < T ? smem_u32(xs + (size_t) ng * KB * 8 + c0) : 0u;
        lx.s1[ng] = 4 * ng + (c1 & 3) < T ? smem_u32(xs + (size_t) ng * KB * 8 + c1) : 0u;
        lx.r0[ng] = lx.r1[ng] = 1.0f;
    }
    return lx;
}

// lane pointers for one expert job over the image of all window rows: column n < 4 = level 1 of row y[n], n >= 4 = level 2
__device__ __forceinline__ LaneX<1> lane_x_job(const uint2* xq, const float* xs, int K, const int* y, int ntok, int lane) {
    LaneX<1> lx;
    const int g = lane >> 2, q = lane & 3, KB = K / 256;
    lx.b[0] = 0u;
    if ((g & 3) < ntok) {
        const int row = y[g & 3];
        lx.b[0] = smem_u32(xq + ((size_t) (row >> 2) * (K / 32) * 8 + (row & 3) + 4 * (g >> 2)) * 4 + q);
    }
    const int c0 = 2 * q, c1 = 2 * q + 1;
    lx.s0[0] = lx.s1[0] = 0u;
    lx.r0[0] = lx.r1[0] = 1.0f;
    if ((c0 & 3) < ntok) {
        const int row = y[c0 & 3];
        lx.s0[0] = smem_u32(xs + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c0 >> 2));
    }
    if ((c1 & 3) < ntok) {
        const int row = y[c1 & 3];
        lx.s1[0] = smem_u32(xs + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c1 >> 2));
    }
    return lx;
}

template <int NG, int SB, bool CHECK>
__device__ __forceinline__ void core_sub_block(const uint32_t (&S0)[5], const uint32_t (&G0)[2], const uint32_t (&S1)[5], const uint32_t (&G1)[2],
                                               uint2 sc0, uint2 sc1, uint32_t table_s, uint32_t lane4, const uint32_t (&bx)[NG],
                                               int (&accI)[NG][4]) {
    const uint32_t a0 = core_decode<2 * SB>(S0, G0, table_s, lane4);
    const uint32_t a2 = core_decode<2 * SB + 1>(S0, G0, table_s, lane4);
    const uint32_t a1 = core_decode<2 * SB>(S1, G1, table_s, lane4);
    const uint32_t a3 = core_decode<2 * SB + 1>(S1, G1, table_s, lane4);
    // sc0 / sc1: the rows' eight scales 1 + 2 s as bytes (even sub-blocks in .x, odd in .y): one byte extract each
    int w0, w1;
    {
        const uint32_t a = SB & 1 ? sc0.y : sc0.x, b = SB & 1 ? sc1.y : sc1.x;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(w0) : "r"(a), "r"(0u), "r"(0x4440u + (SB >> 1)));
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(w1) : "r"(b), "r"(0u), "r"(0x4440u + (SB >> 1)));
    }
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        uint2 b = make_uint2(0u, 0u);
        if (!CHECK || bx[ng]) b = lds_v2<SB * 256>(bx[ng]);   // bx: this lane's cells of the block's first sub-block
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
// CHECK: a zero address in lx means an empty column; without it every address is read (empty rows are zero cells).
// AccT double: the block's four products are exact in double and their sums carry ~2^-53 relative error, so that the
// rounded result does not depend on where a row's K-sum was cut into pieces (expert modes, where the cuts move with the
// number of jobs: a row must give the same bits whatever else is in the window).
template <int NG, bool CHECK = true, typename AccT = float>
__device__ __forceinline__ void core_item(uint32_t tile_s, uint32_t table_s, const LaneX<NG>& lx, int blk, int lane, AccT (&acc)[NG][4]) {
    const int g = lane >> 2;
    const uint32_t lane4 = (uint32_t) lane * 4u;
    const uint32_t a16 = tile_s + lane * 16, a8 = tile_s + lane * 8, a2 = tile_s + lane * 2, ag4 = tile_s + g * 4, ag2 = tile_s + g * 2;
    const uint4 i0 = lds_v4<TILE_IDX>(a16);
    const uint4 i1 = lds_v4<TILE_IDX + 512>(a16);
    const uint2 s0 = lds_v2<TILE_SGN>(a8);
    const uint2 s1 = lds_v2<TILE_SGN + 256>(a8);
    const uint32_t t0 = lds_u16<TILE_TAIL>(a2);
    const uint32_t t1 = lds_u16<TILE_TAIL + 64>(a2);
    const uint32_t sn0 = lds_u32<TILE_SCL>(ag4);
    const uint32_t sn1 = lds_u32<TILE_SCL + 32>(ag4);
    // nibbles -> bytes 1 + 2 s: even sub-blocks (low nibbles) and odd ones (high nibbles)
    const uint2 sc0 = make_uint2((sn0 & 0x0F0F0F0Fu) * 2u + 0x01010101u, ((sn0 >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u);
    const uint2 sc1 = make_uint2((sn1 & 0x0F0F0F0Fu) * 2u + 0x01010101u, ((sn1 >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u);
    const float d0 = __half2float(__ushort_as_half((unsigned short) lds_u16<TILE_D>(ag2)));
    const float d1 = __half2float(__ushort_as_half((unsigned short) lds_u16<TILE_D + 16>(ag2)));
    const uint32_t S0[5] = {i0.x, i0.y, i0.z, i0.w, t0}, S1[5] = {i1.x, i1.y, i1.z, i1.w, t1};
    const uint32_t G0[2] = {s0.x, s0.y}, G1[2] = {s1.x, s1.y};
    uint32_t bx[NG];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) bx[ng] = !CHECK || lx.b[ng] ? lx.b[ng] + (uint32_t) blk * 2048u : 0u;
    int accI[NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int i = 0; i < 4; ++i) accI[ng][i] = 0;
    core_sub_block<NG, 0, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 1, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 2, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 3, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 4, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 5, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 6, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
    core_sub_block<NG, 7, CHECK>(S0, G0, S1, G1, sc0, sc1, table_s, lane4, bx, accI);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        float x0 = !CHECK || lx.s0[ng] ? lds_f32(lx.s0[ng] + (uint32_t) blk * 32u) : 0.f;
        float x1 = !CHECK || lx.s1[ng] ? lds_f32(lx.s1[ng] + (uint32_t) blk * 32u) : 0.f;
        if (!CHECK) {
            x0 *= lx.r0[ng];
            x1 *= lx.r1[ng];
        }
        if constexpr (sizeof(AccT) == 8) {
            acc[ng][0] += (double) (d0 * x0) * (double) accI[ng][0];
            acc[ng][1] += (double) (d0 * x1) * (double) accI[ng][1];
            acc[ng][2] += (double) (d1 * x0) * (double) accI[ng][2];
            acc[ng][3] += (double) (d1 * x1) * (double) accI[ng][3];
        } else {
            acc[ng][0] += d0 * x0 * (float) accI[ng][0];
            acc[ng][1] += d0 * x1 * (float) accI[ng][1];
            acc[ng][2] += d1 * x0 * (float) accI[ng][2];
            acc[ng][3] += d1 * x1 * (float) accI[ng][3];
        }
    }
}

// Quantises 8 consecutive values of one lane (a cell) given the block's maximum over the warp; returns the cells.
// Rounding rides on the FMA pipe: adding 1.5 * 2^23 leaves round-to-nearest-even(x) in the low mantissa bits (its low
// byte is the s8 code), so no value passes through the conversion unit.
__device__ __forceinline__ void core_quant_cell(const float (&x8)[8], float am, uint2& c1, uint2& c2, float& d) {
    constexpr float MAGIC = 12582912.0f;
    d = am * (1.0f / 127.0f);
    const float inv = am > 0.f ? __fdividef(127.0f, am) : 0.f, inv2 = inv * 256.0f;
    uint32_t a8[8], b8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float ta = fmaf(x8[i], inv, MAGIC);              // |x inv| <= 127
        const float af = ta - MAGIC;
        const float tb = fminf(fmaf(fmaf(-af, d, x8[i]), inv2, MAGIC), MAGIC + 127.0f);   // the residue, in steps of d / 256
        a8[i] = __float_as_uint(ta);
        b8[i] = __float_as_uint(tb);
    }
    auto pack = [](uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3) {
        uint32_t lo, hi, r;
        asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(v0), "r"(v1));
        asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(v2), "r"(v3));
        asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(r) : "r"(lo), "r"(hi));
        return r;
    };
    c1 = make_uint2(pack(a8[0], a8[1], a8[2], a8[3]), pack(a8[4], a8[5], a8[6], a8[7]));
    c2 = make_uint2(pack(b8[0], b8[1], b8[2], b8[3]), pack(b8[4], b8[5], b8[6], b8[7]));
}

}  // namespace fnxb

// ------------------------------------------------------------------------------------------------ rows -> image
// A quantisation TASK is one 256-column block of one live row, done by one warp (8 values per lane); a warp works on
// a batch of up to four tasks at once so that their loads and their warp reductions overlap.  quant_fetch() starts a
// task's loads, quant_finish() turns a batch into image cells and scales at (cells, scales) for image rows t (group
// t / 4, column t % 4).  With norm_w the codes are those of x * w and the block's sum of squares goes to
// rs[t * 16 + blk]: the row's 1 / rms (quant_row_factor) multiplies the products later, it is uniform along the row.
// Rows that hold nothing are not tasks: quant_zero_row() clears their cells and scales.
namespace fnxb {
constexpr int QUANT_BATCH = 2;

struct QuantTask {
    const float* src;   // the block's 256 values; null: no task
    int t, blk;
};

// (the block's norm weights ride with the values: one latency, not two)
__device__ __forceinline__ void quant_fetch(const QuantTask& q, const float* norm_w, int lane, float (&v)[8], float (&w)[8]) {
    if (q.src) {
        const float4 a = *reinterpret_cast<const float4*>(q.src + lane * 8), b = *reinterpret_cast<const float4*>(q.src + lane * 8 + 4);
        if (norm_w) {
            const float4 c = *reinterpret_cast<const float4*>(norm_w + q.blk * 256 + lane * 8), d = *reinterpret_cast<const float4*>(norm_w + q.blk * 256 + lane * 8 + 4);
            w[0] = c.x; w[1] = c.y; w[2] = c.z; w[3] = c.w;
            w[4] = d.x; w[5] = d.y; w[6] = d.z; w[7] = d.w;
        }
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

__device__ __forceinline__ void quant_finish(const QuantTask (&q)[QUANT_BATCH], float (&v)[QUANT_BATCH][8], const float (&w)[QUANT_BATCH][8], int K, const float* norm_w, uint2* cells,
                                             float* scales, float* rs, int lane) {
    const int KB = K / 256;
    float am[QUANT_BATCH], ss[QUANT_BATCH];
#pragma unroll
    for (int j = 0; j < QUANT_BATCH; ++j) {
        ss[j] = 0.f;
        if (norm_w && q[j].src) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ss[j] = fmaf(v[j][i], v[j][i], ss[j]);
                v[j][i] *= w[j][i];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < QUANT_BATCH; ++j) {
        am[j] = 0.f;
        if (q[j].src) {
#pragma unroll
            for (int i = 0; i < 8; ++i) am[j] = fmaxf(am[j], fabsf(v[j][i]));
        }
    }
    // the batch's maxima (and sums of squares) cross the warp together: five rounds for all of them
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int j = 0; j < QUANT_BATCH; ++j) {
            am[j] = fmaxf(am[j], __shfl_xor_sync(0xffffffffu, am[j], o));
            if (norm_w) ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], o);
        }
    }
#pragma unroll
    for (int j = 0; j < QUANT_BATCH; ++j)
        if (q[j].src) {
            const int t = q[j].t, blk = q[j].blk, ng = t >> 2, n = t & 3;
            uint2 c1, c2;
            float d;
            core_quant_cell(v[j], am[j], c1, c2, d);
            const int sbG = blk * 8 + (lane >> 2), qq = lane & 3;
            uint2* cell = cells + ((size_t) (ng * (K / 32) + sbG) * 8 + n) * 4 + qq;
            cell[0] = c1;
            cell[16] = c2;
            if (lane == 0) {
                float* sc = scales + (size_t) (ng * KB + blk) * 8;
                sc[n] = d;
                sc[n + 4] = d * (1.0f / 256.0f);
                if (norm_w) rs[t * 16 + blk] = ss[j];
            }
        }
}

// image row t holds nothing: zero cells, zero scales (threads idx of n cooperate)
__device__ __forceinline__ void quant_zero_row(int t, int K, uint2* cells, float* scales, float* rs, int idx, int n_threads) {
    const int KB = K / 256, ng = t >> 2, n = t & 3;
    for (int i = idx; i < (K / 32) * 8; i += n_threads) {   // (sub-block, level, q)
        const int sbG = i >> 3, lvl = (i >> 2) & 1, q = i & 3;
        cells[((size_t) (ng * (K / 32) + sbG) * 8 + n + 4 * lvl) * 4 + q] = make_uint2(0u, 0u);
    }
    for (int i = idx; i < KB * 2; i += n_threads) scales[(size_t) (ng * KB + (i >> 1)) * 8 + n + 4 * (i & 1)] = 0.f;
    for (int i = idx; i < KB; i += n_threads) rs[t * 16 + i] = 0.f;
}

// 1 / rms of image row t from the block sums (after the barrier that follows the tasks)
__device__ __forceinline__ float quant_row_factor(const float* rs, int t, int K, float eps) {
    float ss = 0.f;
    for (int c = 0; c < K / 256; ++c) ss += rs[t * 16 + c];
    return rsqrtf(ss / (float) K + eps);
}
}  // namespace fnxb

// ------------------------------------------------------------------------------------------------ streaming by warp
// The product is a sequence of ITEMS: one 16-row x 256-column tile block against the activation cells.  A unit is a
// 16-row tile across all of K (gate|up: the gate tile then its up tile): nbu consecutive items whose weights are one
// contiguous run of tile blocks (two runs for gate|up).  A block's items are dealt to its warps in equal contiguous
// shares, so every warp has the same amount of decode work whatever the number of units.  Each warp streams its
// items through its PRIVATE ring of bulk async copies (lane 0 issues, every lane waits on the slot's mbarrier) and
// accumulates in registers.  A unit that lies wholly inside one warp's share is finished and written by that warp;
// a unit cut by share boundaries leaves its pieces in shared memory, and after ONE block barrier the warp that
// holds the unit's first piece adds the others in warp order and writes it.  Nothing else in the loop is
// block-wide: no per-step barrier, no thread that issues copies for others.
namespace fnxb {

enum { MAT_DENSE = 0, MAT_GATEUP = 1, MAT_DOWN = 2 };

// accumulator of a row's K-sum: the dense product is cut the same way for any number of rows (float, summed in a fixed
// order); the expert products are cut where the job count puts the warps' shares (double, see core_item)
template <int MODE>
struct MatAcc {
    using type = double;
};
template <>
struct MatAcc<MAT_DENSE> {
    using type = float;
};

struct MatDesc {
    const uint8_t* W;        // the dense matrix, or expert 0 of the experts held at W
    size_t expert_stride;
    int e_base;              // first expert held at W
    const uint8_t* Wsh;      // the shared expert (job.w >= E)
    int E;
    const fnx_job* jobs;     // null: one dense job
    const uint8_t* const* jobw;   // jobs mode: weight base of job (j - jobw0), in shared memory
    int jobw0;
    int rows, K;             // output rows per job (gate|up: F)
    float* out;
    int ldo, accumulate;
};

// fixed-point image of a float addend: integer sums do not depend on the order of their terms, so rows summed in any
// order (a loop, several kernels, expert-parallel ranks) give the same bits
constexpr float FIX_SCALE = 4294967296.0f;            // 2^32
constexpr double FIX_INV = 1.0 / 4294967296.0;
__device__ __forceinline__ unsigned long long fix_from_float(float v) { return (unsigned long long) __float2ll_rn(v * FIX_SCALE); }
__device__ __forceinline__ float fix_to_float(unsigned long long a) { return (float) ((double) (long long) a * FIX_INV); }

struct WarpRing {
    uint8_t* slots;          // R x TILE_BYTES
    uint32_t slots_s;        // their shared address
    uint64_t* bars;          // one per slot (up to 8)
    int R;                   // slots in use: may change while the ring is empty
    unsigned in_slot, out_slot;   // next slot to fill, next slot to read
    unsigned parity;         // bit i: the phase parity slot i's next read waits for
    int pre;                 // items of the next mat_items() call already issued (mat_preissue)
    // the issue cursor (lane 0): next item `ahead` = block ab of local tile al of job aj, weights aw
    int ahead, ab, al, aj;
    const uint8_t* aw;
    const uint8_t* asrc;     // the next item's tile block
};

__device__ __forceinline__ void ring_reset(WarpRing& r, int R) {
    r.R = R;
    r.in_slot = r.out_slot = 0;
    r.pre = 0;
}

// a piece of a unit left for the end-of-pass combine: slot [warp][0] = a piece that continues a unit begun by an
// earlier warp, slot [warp][1] = the first piece of a unit that later warps continue
template <int NG, int MODE>
struct PieceSlotT {
    int unit;                // -1: none, -2: the warp had no items at all
    int b_lo, b_hi, job, ntok;
    int orow[4 * NG];
    double v[(MODE == 1 ? 2 : 1) * NG * 64];   // [kind (gate|up only: 0 gate, 1 up)][group][16 lanes][4]   (MODE 1 = MAT_GATEUP)
};

__device__ __forceinline__ int mat_blocks_per_unit(int mode, int K) { return mode == MAT_GATEUP ? 2 * (K / 256) : K / 256; }

// weight base of job j: the dense matrix, or the job's expert (from the per-pass table when there is one)
__device__ __forceinline__ const uint8_t* mat_job_weights(const MatDesc& m, int j) {
    if (!m.jobs) return m.W;
    if (m.jobw) return m.jobw[j - m.jobw0];
    const int e = m.jobs[j].w;
    return e >= m.E ? m.Wsh : m.W + (size_t) (e - m.e_base) * m.expert_stride;
}

// the 16 x rows results of unit (job rows orow, local tile lu) from this lane's sums (threads q < 2 hold them)
template <int NG, int MODE, typename AccT>
__device__ __forceinline__ void mat_write_unit(const MatDesc& m, int lu, const int (&orow)[4 * NG], int ntok, int lane, const AccT (&gacc)[NG][4],
                                               const AccT (&acc)[NG][4]) {
    const int g = lane >> 2, q = lane & 3;
    if (q >= 2) return;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int tok = 4 * ng + 2 * q + (k & 1), row = lu * 16 + g + 8 * (k >> 1);
            if (tok < ntok) {
                const float v = MODE == MAT_GATEUP ? siluf_((float) gacc[ng][k]) * (float) acc[ng][k] : (float) acc[ng][k];
                float* dst = m.out + (size_t) orow[tok] * m.ldo + row;
                *dst = m.accumulate ? *dst + v : v;
            }
        }
}

// places the warp's issue cursor at the first item of its share of units [ua, ub)
template <int MODE>
__device__ __forceinline__ void mat_cursor(const MatDesc& m, int ua, int ub, WarpRing& ring, int warp, int nwarp) {
    const int nbu = mat_blocks_per_unit(MODE, m.K), upj = m.rows / 16;
    const unsigned N = (unsigned) (ub - ua) * nbu;   // < 2^26 for any matrix here
    const int i0 = (int) (N * warp / nwarp), i1 = (int) (N * (warp + 1) / nwarp);
    ring.ahead = i0;
    ring.ab = i0 % nbu;
    ring.al = (ua + i0 / nbu) % upj;
    ring.aj = (ua + i0 / nbu) / upj;
    ring.aw = i0 < i1 ? mat_job_weights(m, ring.aj) : nullptr;
    const int KB = m.K / 256;
    ring.asrc = MODE == MAT_GATEUP && ring.ab >= KB ? ring.aw + ((size_t) (upj + ring.al) * KB + (ring.ab - KB)) * TILE_BYTES
                                                    : ring.aw + ((size_t) ring.al * KB + ring.ab) * TILE_BYTES;
}

// lane 0: bulk copies for the items before min(i1, limit) that are not yet on their way
template <int MODE>
__device__ __forceinline__ void mat_issue_upto(const MatDesc& m, WarpRing& ring, int i1, int limit, int lane) {
    if (lane != 0) return;
    const int KB = m.K / 256, nbu = mat_blocks_per_unit(MODE, m.K), upj = m.rows / 16;
    while (ring.ahead < i1 && ring.ahead < limit) {
        const unsigned st = ring.in_slot;
        // the slot's previous readers are ordered before this copy by the warp barrier that precedes the call
        mbar_expect_tx(&ring.bars[st], TILE_BYTES);
        bulk_g2s(ring.slots + (size_t) st * TILE_BYTES, ring.asrc, TILE_BYTES, &ring.bars[st]);
        ring.in_slot = st + 1 == (unsigned) ring.R ? 0u : st + 1;
        ++ring.ahead;
        ring.asrc += TILE_BYTES;   // a tile's blocks, and a matrix's tiles, follow one another
        ++ring.ab;
        if (MODE == MAT_GATEUP && ring.ab == KB) ring.asrc = ring.aw + (size_t) (upj + ring.al) * KB * TILE_BYTES;
        if (ring.ab == nbu) {
            ring.ab = 0;
            if (++ring.al == upj) {
                ring.al = 0;
                ++ring.aj;
                if (ring.ahead < i1) ring.aw = mat_job_weights(m, ring.aj);
            }
            if (MODE == MAT_GATEUP || ring.al == 0) ring.asrc = ring.aw + (size_t) ring.al * KB * TILE_BYTES;
        }
    }
}

// before the barrier that precedes a matrix phase whose weights do not depend on it: the warp's first items on their way
// (`depth` copies per warp: the copy engine takes a request every ~80 cycles per SM, and a full ring of requests from
// every warp at once would hold the issuing lanes for microseconds)
template <int MODE>
__device__ __forceinline__ void mat_preissue(const MatDesc& m, int ua, int ub, WarpRing& ring, int warp, int nwarp, int lane, int depth) {
    const int nbu = mat_blocks_per_unit(MODE, m.K);
    const unsigned N = (unsigned) (ub - ua) * nbu;   // < 2^26 for any matrix here
    const int i0 = (int) (N * warp / nwarp), i1 = (int) (N * (warp + 1) / nwarp);
    mat_cursor<MODE>(m, ua, ub, ring, warp, nwarp);
    mat_issue_upto<MODE>(m, ring, i1, i0 + min(ring.R, depth), lane);
    ring.pre = 1;
}

// This warp's share of the items of units [ua, ub).  `lane_x(j, lx, ntok, orow)` sets the lane's activation pointers
// and output rows for job j.  pieces: [nwarp][2] slots.  Returns false when a wait gave up.  The caller runs a block
// barrier and then mat_combine().
template <int NG, int MODE, typename LaneXFn>
__device__ __forceinline__ bool mat_items(const MatDesc& m, int ua, int ub, uint32_t table_s, WarpRing& ring, PieceSlotT<NG, MODE>* pieces, int warp,
                                          int nwarp, int lane, LaneXFn&& lane_x) {
    const int KB = m.K / 256, nbu = mat_blocks_per_unit(MODE, m.K), upj = m.rows / 16;
    const unsigned N = (unsigned) (ub - ua) * nbu;   // < 2^26 for any matrix here
    const int i0 = (int) (N * warp / nwarp), i1 = (int) (N * (warp + 1) / nwarp);
    PieceSlotT<NG, MODE>* mine = pieces + warp * 2;
    if (lane == 0) {
        mine[0].unit = i0 < i1 ? -1 : -2;
        mine[1].unit = -1;
    }
    if (!ring.pre) mat_cursor<MODE>(m, ua, ub, ring, warp, nwarp);
    ring.pre = 0;
    auto issue_upto = [&](int limit) { mat_issue_upto<MODE>(m, ring, i1, limit, lane); };
    issue_upto(i0 + ring.R);
    int cur_job = -1, ntok = 0, b_lo = 0;
    int orow[4 * NG];
    LaneX<NG> lx;
    using AccT = typename MatAcc<MODE>::type;
    AccT acc[NG][4], gacc[NG][4];
    int b = i0 % nbu, lu = (ua + i0 / nbu) % upj, j = (ua + i0 / nbu) / upj;
    for (int s = i0; s < i1; ++s) {
        if (b == 0 || s == i0) {
            b_lo = b;
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[ng][k] = gacc[ng][k] = 0;
            if (j != cur_job) {
                cur_job = j;
                lane_x(j, lx, ntok, orow);
            }
        }
        const unsigned st = ring.out_slot;
        if (!mbar_wait_bounded(&ring.bars[st], (ring.parity >> st) & 1u, 8000000u)) return false;
        ring.parity ^= 1u << st;
        ring.out_slot = st + 1 == (unsigned) ring.R ? 0u : st + 1;
        const uint32_t tile_s = ring.slots_s + st * (uint32_t) TILE_BYTES;
        if (MODE == MAT_GATEUP && b < KB) core_item<NG, false, AccT>(tile_s, table_s, lx, b, lane, gacc);
        else core_item<NG, false, AccT>(tile_s, table_s, lx, MODE == MAT_GATEUP ? b - KB : b, lane, acc);
        __syncwarp();
        issue_upto(s + 1 + ring.R);
        if (b == nbu - 1 || s == i1 - 1) {
            // level 1 (threads q = 0, 1) + level 2 (q = 2, 3) of the same rows
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[ng][k] += __shfl_xor_sync(0xffffffffu, acc[ng][k], 2);
                    if (MODE == MAT_GATEUP) gacc[ng][k] += __shfl_xor_sync(0xffffffffu, gacc[ng][k], 2);
                }
            if (b_lo == 0 && b == nbu - 1) {
                mat_write_unit<NG, MODE, AccT>(m, lu, orow, ntok, lane, gacc, acc);
            } else {
                PieceSlotT<NG, MODE>* ps = mine + (b_lo == 0 ? 1 : 0);
                if (lane == 0) {
                    ps->unit = j * upj + lu;
                    ps->b_lo = b_lo;
                    ps->b_hi = b + 1;
                    ps->job = j;
                    ps->ntok = ntok;
#pragma unroll
                    for (int i = 0; i < 4 * NG; ++i) ps->orow[i] = orow[i];
                }
                if ((lane & 3) < 2) {
                    const int l16 = (lane >> 2) * 2 + (lane & 3);
#pragma unroll
                    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (MODE == MAT_GATEUP) {
                                ps->v[(ng * 16 + l16) * 4 + k] = gacc[ng][k];
                                ps->v[((NG + ng) * 16 + l16) * 4 + k] = acc[ng][k];
                            } else {
                                ps->v[(ng * 16 + l16) * 4 + k] = acc[ng][k];
                            }
                        }
                }
            }
        }
        if (++b == nbu) {
            b = 0;
            if (++lu == upj) {
                lu = 0;
                ++j;
            }
        }
    }
    return true;
}

// after the block barrier: the warp that holds a unit's first piece adds the later warps' pieces and writes the unit
template <int NG, int MODE>
__device__ __forceinline__ void mat_combine(const MatDesc& m, const PieceSlotT<NG, MODE>* pieces, int warp, int nwarp, int lane) {
    const PieceSlotT<NG, MODE>* first = pieces + warp * 2 + 1;
    const int u = first->unit;
    if (u < 0) return;
    const int nbu = mat_blocks_per_unit(MODE, m.K), upj = m.rows / 16;
    const int l16 = (lane >> 2) * 2 + (lane & 3);
    const bool holder = (lane & 3) < 2;
    using AccT = typename MatAcc<MODE>::type;
    AccT acc[NG][4], gacc[NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            gacc[ng][k] = holder && MODE == MAT_GATEUP ? (AccT) first->v[(ng * 16 + l16) * 4 + k] : (AccT) 0;
            acc[ng][k] = holder ? (AccT) first->v[((MODE == MAT_GATEUP ? NG + ng : ng) * 16 + l16) * 4 + k] : (AccT) 0;
        }
    for (int ww = warp + 1; ww < nwarp; ++ww) {
        const PieceSlotT<NG, MODE>* c = pieces + ww * 2;
        if (c->unit == -2) continue;
        if (c->unit != u) break;
#pragma unroll
        for (int ng = 0; ng < NG; ++ng)
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (holder) {
                    if (MODE == MAT_GATEUP) gacc[ng][k] += (AccT) c->v[(ng * 16 + l16) * 4 + k];
                    acc[ng][k] += (AccT) c->v[((MODE == MAT_GATEUP ? NG + ng : ng) * 16 + l16) * 4 + k];
                }
        if (c->b_hi == nbu) break;
    }
    int orow[4 * NG];
#pragma unroll
    for (int i = 0; i < 4 * NG; ++i) orow[i] = first->orow[i];
    mat_write_unit<NG, MODE, AccT>(m, u % upj, orow, first->ntok, lane, gacc, acc);
}

}  // namespace fnxb
