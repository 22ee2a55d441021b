// IQ3_S matrix x few activation rows: the one kernel behind the dense projections (q/k/v/o, qkvz, ssm_out, head,
// MTP fc) and the routed/shared experts (gate|up + SwiGLU, down).
//
// Replaces the reference's decode-path quantised GEMVs: k_mmvq (engine/src/kernels.cu:192-228), k_q8s
// (engine/src/dense.cuh:211), k_moe_gu / k_moe_down (engine/src/moe.cuh:572-658) and the P100 lane-per-row
// kernel k_moe_rows (engine/src/p100_moe_rows.cuh:266-342).  Like the reference it multiplies integer codebook
// magnitudes by int8 activations and applies the scales afterwards; unlike it
//   - the weight stream is staged through shared memory by bulk async copies (28,160-byte steps, 3 in flight per
//     SM) from the tile layout of iq3s_tile.h, so every global read is a full, aligned burst;
//   - the codebook lives in shared memory 32 times, once per bank, so the 9-bit lookups never conflict;
//   - activations are quantised to two int8 levels per 256-column block (x ~ d (q1 + q2 / 256), error
//     <= amax / 65024), and both levels of up to 4 rows ride in the 8 columns of one mma.sync.m16n8k32.s8, so a
//     decoded weight fragment is used for every row at once and the result is fp16-class accurate;
//   - a persistent grid of one CTA per SM walks a contiguous range of steps of the whole job list.
//
// Per-weight work is what bounds this kernel (about 2 integer instructions per weight besides the loads): the
// byte stream itself is 110 bytes per 256 weights.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fnx_common.cuh"
#include "iq3s_grid.h"
#include "iq3s_tile.h"

namespace fnxb {

__device__ const uint32_t g_iq3s_grid[512] = {FNX_IQ3S_GRID_VALUES};

// Phase stamps (the reference's FNX_PROF idea, engine/src/engine.cu:1382-1529): when a buffer is registered, thread 0 of
// every block writes %globaltimer at its phase boundaries: [block][MMV_PROF_SLOTS] u64, slot 0 = how many were written.
constexpr int MMV_PROF_SLOTS = 64;
__device__ unsigned long long* g_mmv_prof = nullptr;
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define MMV_STAMP()                                                                         \
    do {                                                                                    \
        if (prof && tid == 0 && nstamp < MMV_PROF_SLOTS - 1) prof[1 + nstamp++] = gtime(); \
    } while (0)

enum { MMV_DENSE = 0, MMV_GATEUP = 1, MMV_DOWN = 2 };
constexpr int MMV_THREADS = 512, MMV_WARPS = 16, MMV_ITEMS = 16;
constexpr int MMV_STEP_BYTES = MMV_ITEMS * TILE_BYTES;   // 28,160
constexpr int MMV_TABLE_BYTES = 512 * 128;

struct MmvParams {
    const uint8_t* W;
    size_t expert_stride;
    int e_base;
    const uint8_t* Wsh;
    int E;
    const fnx_job* jobs;
    const int* njobs;
    int njobs_max;
    int T;
    const float* x;
    int ldx;
    const float* norm_w;
    float eps;
    float* out;
    int ldo;
    int rows;   // output rows per job (gate|up: F)
    int K;
    int accumulate;
    int nstage;
    unsigned* err;
};

struct MmvSmem {
    uint8_t* table;
    uint8_t* stage;
    uint2* xq;
    float* xs;
    float* part;
    float* rs;
    uint64_t* bars;
};

__host__ __device__ inline size_t mmv_smem_bytes(int K, int NG, int nstage) {
    size_t b = MMV_TABLE_BYTES;
    b += (size_t) nstage * MMV_STEP_BYTES;
    b += (size_t) NG * (K / 32) * 32 * sizeof(uint2);       // xq
    b += (size_t) NG * (K / 256) * 8 * sizeof(float);       // xs
    b += (size_t) 2 * MMV_ITEMS * 16 * 4 * NG * sizeof(float);   // part, double buffered
    b += 32 * sizeof(float);                                // rs: square sums per (row slot, chunk)
    b += 8 * sizeof(uint64_t);                              // barriers (one per stage, at most 8)
    return b;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// four s32 -> four saturated s8 in one word (byte 0 = a)
__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}

template <int I>
__device__ __forceinline__ uint32_t decode_group(const uint32_t (&S)[5], const uint32_t (&G)[2], const uint8_t* table, uint32_t lane4) {
    // (field & 0xFF80) | 4 lane: one logic op, then a shared load off the table's (uniform) base
    const uint32_t off = tile_field<I>(S) | lane4;
    const uint32_t mag = *reinterpret_cast<const uint32_t*>(table + off);
    return tile_apply_sign(mag, tile_sign_mask<I>(G));
}

// One item: a 16-row x 256-column tile against this block's activation cells; adds into acc[ng][0..3] =
// (row g, col 2q), (row g, col 2q+1), (row g+8, col 2q), (row g+8, col 2q+1), columns = 4 rows x 2 levels.
template <int NG, int SB>
__device__ __forceinline__ void item_sub_block(const uint32_t (&S0)[5], const uint32_t (&G0)[2], const uint32_t (&S1)[5],
                                               const uint32_t (&G1)[2], uint32_t sc0, uint32_t sc1, const uint8_t* table, uint32_t lane4,
                                               const uint2* xq_blk, int xq_group_stride, int lane, int (&accI)[NG][4]) {
    const uint32_t a0 = decode_group<2 * SB>(S0, G0, table, lane4);
    const uint32_t a2 = decode_group<2 * SB + 1>(S0, G0, table, lane4);
    const uint32_t a1 = decode_group<2 * SB>(S1, G1, table, lane4);
    const uint32_t a3 = decode_group<2 * SB + 1>(S1, G1, table, lane4);
    const int w0 = 1 + 2 * (int) ((sc0 >> (4 * SB)) & 15u), w1 = 1 + 2 * (int) ((sc1 >> (4 * SB)) & 15u);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        const uint2 b = xq_blk[ng * xq_group_stride + SB * 32 + lane];
        int c[4];
        mma_s8(c, a0, a1, a2, a3, b.x, b.y);
        accI[ng][0] += w0 * c[0];
        accI[ng][1] += w0 * c[1];
        accI[ng][2] += w1 * c[2];
        accI[ng][3] += w1 * c[3];
    }
}

template <int NG>
__device__ __forceinline__ void mmv_item(const uint8_t* tile, const uint8_t* table, const uint2* xq_blk, int xq_group_stride,
                                         const float* xs_blk, int xs_group_stride, int lane, float (&acc)[NG][4]) {
    const int g = lane >> 2, q = lane & 3;
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
    item_sub_block<NG, 0>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 1>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 2>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 3>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 4>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 5>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 6>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
    item_sub_block<NG, 7>(S0, G0, S1, G1, sc0, sc1, table, lane4, xq_blk, xq_group_stride, lane, accI);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        const float2 xsc = *reinterpret_cast<const float2*>(xs_blk + ng * xs_group_stride + 2 * q);
        acc[ng][0] += d0 * xsc.x * (float) accI[ng][0];
        acc[ng][1] += d0 * xsc.y * (float) accI[ng][1];
        acc[ng][2] += d1 * xsc.x * (float) accI[ng][2];
        acc[ng][3] += d1 * xsc.y * (float) accI[ng][3];
    }
}

// Quantises the job's activation rows into the MMA's B layout: cell (sub-block sbG, column n, thread q) = the 8
// int8 values x[32 sbG + 8 q .. + 7] of row n (columns 0..3: level 1 of rows 0..3, columns 4..7: level 2).
// A task = (row slot, chunk of up to 4 blocks): a warp issues all of a task's loads at once, so the whole prologue
// costs one or two memory latencies.  With an RMS norm the row's scalar 1 / rms multiplies every value, so the
// int8 codes are those of x * w and only the block scales take the factor, after the row's square sum is known.
template <int NG, int MODE>
__device__ __forceinline__ void mmv_load_x(const MmvParams& p, const MmvSmem& sm, const int* xrow, int ntok, int tid) {
    const int warp = tid >> 5, lane = tid & 31, KB = p.K / 256, nslot = 4 * NG;
    const int CB = KB < 4 ? KB : 4, nchunk = KB / CB;   // blocks per chunk, chunks per row
    const bool norm = MODE != MMV_DOWN && p.norm_w != nullptr;
    for (int task = warp; task < nslot * nchunk; task += MMV_WARPS) {
        const int ts = task / nchunk, ck = task % nchunk, ng = ts >> 2, n = ts & 3;
        const bool live = ts < ntok;
        float4 v[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < CB) {
                v[j][0] = v[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) {
                    const float* xr = p.x + (size_t) xrow[ts] * p.ldx + (ck * CB + j) * 256 + lane * 8;
                    v[j][0] = *reinterpret_cast<const float4*>(xr);
                    v[j][1] = *reinterpret_cast<const float4*>(xr + 4);
                }
            }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < CB) {
                const int blk = ck * CB + j;
                float x8[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w, v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
                if (norm) {
                    const float* w = p.norm_w + blk * 256 + lane * 8;
                    const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
                    const float w8[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        ss = fmaf(x8[i], x8[i], ss);
                        x8[i] *= w8[i];
                    }
                }
                float am = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(x8[i]));
                am = warp_max(am);
                const float d = am / 127.0f, inv = am > 0.f ? 127.0f / am : 0.f, inv2 = inv * 256.0f;
                int a8[8], b8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    a8[i] = __float2int_rn(x8[i] * inv);                              // |a| <= 127 by construction
                    b8[i] = __float2int_rn((x8[i] - (float) a8[i] * d) * inv2);       // |b| <= 128: saturated when packed
                }
                const uint32_t lo1 = pack_s8x4(a8[0], a8[1], a8[2], a8[3]), hi1 = pack_s8x4(a8[4], a8[5], a8[6], a8[7]);
                const uint32_t lo2 = pack_s8x4(b8[0], b8[1], b8[2], b8[3]), hi2 = pack_s8x4(b8[4], b8[5], b8[6], b8[7]);
                const int sbG = blk * 8 + (lane >> 2), q = lane & 3;
                uint2* c1 = sm.xq + ((size_t) (ng * (p.K / 32) + sbG) * 8 + n) * 4 + q;
                c1[0] = make_uint2(lo1, hi1);
                c1[16] = make_uint2(lo2, hi2);   // column n + 4
                if (lane == 0) {
                    float* xs = sm.xs + (size_t) (ng * KB + blk) * 8;
                    xs[n] = d;
                    xs[n + 4] = d * (1.0f / 256.0f);
                }
            }
        if (norm) {
            ss = warp_sum(ss);
            if (lane == 0) sm.rs[ts * 4 + ck] = ss;
        }
    }
    __syncthreads();
    if (norm) {
        for (int i = tid; i < ntok * KB; i += MMV_THREADS) {
            const int ts = i / KB, blk = i % KB, ng = ts >> 2, n = ts & 3;
            float ss = 0.f;
            for (int c = 0; c < nchunk; ++c) ss += sm.rs[ts * 4 + c];
            const float r = rsqrtf(ss / (float) p.K + p.eps);
            float* xs = sm.xs + (size_t) (ng * KB + blk) * 8;
            xs[n] *= r;
            xs[n + 4] *= r;
        }
        __syncthreads();
    }
}

template <int NG, int MODE>
__global__ void __launch_bounds__(MMV_THREADS, 1) k_iq3s_mmv(const MmvParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = p.K / 256, TPS = MMV_ITEMS / KB, NST = p.nstage;
    MmvSmem sm;
    {
        uint8_t* b = smem_raw;
        sm.table = b; b += MMV_TABLE_BYTES;
        sm.stage = b; b += (size_t) NST * MMV_STEP_BYTES;
        sm.xq = reinterpret_cast<uint2*>(b); b += (size_t) NG * (p.K / 32) * 32 * sizeof(uint2);
        sm.xs = reinterpret_cast<float*>(b); b += (size_t) NG * KB * 8 * sizeof(float);
        sm.part = reinterpret_cast<float*>(b); b += (size_t) 2 * MMV_ITEMS * 16 * 4 * NG * sizeof(float);
        sm.rs = reinterpret_cast<float*>(b); b += 32 * sizeof(float);
        sm.bars = reinterpret_cast<uint64_t*>(b);
    }
    unsigned long long* prof = g_mmv_prof ? g_mmv_prof + (size_t) blockIdx.x * MMV_PROF_SLOTS : nullptr;
    int nstamp = 0;
    MMV_STAMP();
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < NST; ++i) mbar_init(&sm.bars[i], 1);
        fence_barrier_init();
    }
    // steps of one job: gate|up walks h-tiles (TPS / 2 per step), the others row tiles (TPS per step)
    const int spj = MODE == MMV_GATEUP ? p.rows / (8 * TPS) : p.rows / (16 * TPS);
    int njobs = 1, s0 = 0, s1 = 0;
    auto job_weights = [&](int j) -> const uint8_t* {
        if (!p.jobs) return p.W;
        const int e = p.jobs[j].w;
        return e >= p.E ? p.Wsh : p.W + (size_t) (e - p.e_base) * p.expert_stride;
    };
    auto issue = [&](int s) {   // one thread: stage the weights of global step s
        const int j = s / spj, ls = s % spj, st = (s - s0) % NST;
        const uint8_t* W = job_weights(j);
        uint8_t* dst = sm.stage + (size_t) st * MMV_STEP_BYTES;
        mbar_expect_tx(&sm.bars[st], MMV_STEP_BYTES);
        if (MODE == MMV_GATEUP) {
            const size_t half = (size_t) MMV_STEP_BYTES / 2;   // TPS / 2 gate tiles, then their up tiles
            bulk_g2s(dst, W + (size_t) ls * half, (unsigned) half, &sm.bars[st]);
            bulk_g2s(dst + half, W + (size_t) (p.rows / 16) * KB * TILE_BYTES + (size_t) ls * half, (unsigned) half, &sm.bars[st]);
        } else {
            bulk_g2s(dst, W + (size_t) ls * MMV_STEP_BYTES, MMV_STEP_BYTES, &sm.bars[st]);
        }
    };
    auto plan = [&]() {
        const long long total = (long long) njobs * spj;
        s0 = (int) (total * blockIdx.x / gridDim.x);
        s1 = (int) (total * (blockIdx.x + 1) / gridDim.x);
    };
    // a dense matrix is the same whatever ran before: its first steps are on their way before anything else
    if (MODE == MMV_DENSE && !p.jobs) {
        plan();
        if (tid == 0)
            for (int i = 0; i < NST && s0 + i < s1; ++i) issue(s0 + i);
    }
    // the codebook, one copy per bank: entry e at byte e * 128 + 4 * lane
    for (int e = tid; e < 512; e += MMV_THREADS) {
        const uint32_t v = g_iq3s_grid[e];
        uint4* d = reinterpret_cast<uint4*>(sm.table + e * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = make_uint4(v, v, v, v);
    }
    pdl_wait();   // from here on: what earlier kernels of the stream wrote (activations, job lists)
    __syncthreads();
    MMV_STAMP();
    if (!(MODE == MMV_DENSE && !p.jobs)) {
        njobs = p.jobs ? min(*p.njobs, p.njobs_max) : 1;
        plan();
        if (tid == 0)
            for (int i = 0; i < NST && s0 + i < s1; ++i) issue(s0 + i);
    }
    if (s0 >= s1) return;

    const int xq_gs = (p.K / 32) * 32, xs_gs = KB * 8;
    int cur_job = -1, ntok = 0;
    int xrow[4 * NG], orow[4 * NG];
    bool ok = true;
    for (int s = s0; s < s1; ++s) {
        const int j = s / spj, ls = s % spj, st = (s - s0) % NST, buf = (s - s0) & 1;
        if (j != cur_job) {
            cur_job = j;
            if (p.jobs) {
                const fnx_job jb = p.jobs[j];
                ntok = min(jb.n, 4 * NG);
#pragma unroll
                for (int i = 0; i < 4 * NG; ++i) {
                    xrow[i] = MODE == MMV_DOWN ? jb.out[i & 3] : jb.y[i & 3];
                    orow[i] = jb.out[i & 3];
                }
            } else {
                ntok = p.T;
#pragma unroll
                for (int i = 0; i < 4 * NG; ++i) xrow[i] = orow[i] = i;
            }
            mmv_load_x<NG, MODE>(p, sm, xrow, ntok, tid);
            MMV_STAMP();
        }
        if (!mbar_wait_bounded(&sm.bars[st], ((s - s0) / NST) & 1)) {
            ok = false;
            break;
        }
        MMV_STAMP();
        const uint8_t* stage = sm.stage + (size_t) st * MMV_STEP_BYTES;
        float* part = sm.part + (size_t) buf * MMV_ITEMS * 16 * 4 * NG;
        {
            const int it = warp, blk = it % KB;
            float acc[NG][4];
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[ng][i] = 0.f;
            mmv_item<NG>(stage + (size_t) it * TILE_BYTES, sm.table, sm.xq + (size_t) blk * 8 * 32, xq_gs, sm.xs + blk * 8, xs_gs, lane, acc);
            // level 1 (threads q = 0, 1) + level 2 (q = 2, 3) of the same rows
            const int g = lane >> 2, q = lane & 3;
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[ng][i] += __shfl_xor_sync(0xffffffffu, acc[ng][i], 2);
                if (q < 2) {
                    float* pr = part + ((size_t) it * 16 + g) * (4 * NG) + ng * 4 + 2 * q;
                    *reinterpret_cast<float2*>(pr) = make_float2(acc[ng][0], acc[ng][1]);
                    *reinterpret_cast<float2*>(pr + 8 * 4 * NG) = make_float2(acc[ng][2], acc[ng][3]);
                }
            }
        }
        __syncthreads();
        MMV_STAMP();
        if (tid == 0 && s + NST < s1) {
            fence_proxy_async();
            issue(s + NST);
        }
        // the step's outputs: sums over the K blocks in block order
        if (MODE == MMV_GATEUP) {
            const int HPS = TPS / 2;   // h-tiles in the step; items [0, 8) gate tiles, [8, 16) up tiles
            for (int o = tid; o < HPS * 16 * ntok; o += MMV_THREADS) {
                const int tok = o / (HPS * 16), rr = o % (HPS * 16), tl = rr / 16, r = rr % 16;
                float gs = 0.f, us = 0.f;
                for (int b = 0; b < KB; ++b) {
                    gs += part[((size_t) (tl * KB + b) * 16 + r) * (4 * NG) + tok];
                    us += part[((size_t) (8 + tl * KB + b) * 16 + r) * (4 * NG) + tok];
                }
                p.out[(size_t) orow[tok] * p.ldo + (size_t) ls * HPS * 16 + rr] = siluf_(gs) * us;
            }
        } else {
            for (int o = tid; o < TPS * 16 * ntok; o += MMV_THREADS) {
                const int tok = o / (TPS * 16), rr = o % (TPS * 16), tl = rr / 16, r = rr % 16;
                float sum = 0.f;
                for (int b = 0; b < KB; ++b) sum += part[((size_t) (tl * KB + b) * 16 + r) * (4 * NG) + tok];
                float* dst = p.out + (size_t) orow[tok] * p.ldo + (size_t) ls * TPS * 16 + rr;
                *dst = p.accumulate ? *dst + sum : sum;
            }
        }
    }
    MMV_STAMP();
    if (prof && tid == 0) prof[0] = (unsigned long long) nstamp;
    if (!ok) {
        if (tid == 0) atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
        // give this CTA's copies still in flight a bounded chance to land before its shared memory is released
        for (int i = 0; i < NST; ++i) mbar_wait_bounded(&sm.bars[i], 0, 100000u);
    }
}

template <int NG, int MODE>
static int launch_mmv(const MmvParams& p0, cudaStream_t st) {
    MmvParams p = p0;
    const int KB = p.K / 256;
    p.nstage = 4;   // as many 28 KB steps in flight as the shared memory left by the codebook and the activations holds
    size_t smem = mmv_smem_bytes(p.K, NG, p.nstage);
    while (smem > 227 * 1024 && p.nstage > 2) {
        --p.nstage;
        smem = mmv_smem_bytes(p.K, NG, p.nstage);
    }
    if (smem > 227 * 1024) return fail(FNX_E_ARG, "iq3s_mmv: %d columns x %d rows need %zu bytes of shared memory", p.K, 4 * NG, smem);
    (void) KB;
    static bool configured = false;
    if (!configured) {
        FNX_CUDA_OK(cudaFuncSetAttribute(k_iq3s_mmv<NG, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured = true;
    }
    {
        const cudaError_t le_ = launch_k(k_iq3s_mmv<NG, MODE>, dim3(sm_count()), dim3(MMV_THREADS), smem, st, p);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "iq3s_mmv: launch failed: %s", cudaGetErrorString(le_));
    }
    return FNX_OK;
}

static int check_cols(int cols) {
    if (cols != 256 && cols != 512 && cols != 1024 && cols != 2048 && cols != 4096)
        return fail(FNX_E_ARG, "iq3s_mmv: %d columns (256, 512, 1024, 2048 or 4096)", cols);
    return FNX_OK;
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_debug_profile_buffer(void* dev_u64) {
    unsigned long long* p = (unsigned long long*) dev_u64;
    FNX_CUDA_OK(cudaMemcpyToSymbol(g_mmv_prof, &p, sizeof p));
    return FNX_OK;
}

extern "C" int fnx_dense(const void* W, int rows, int cols, const float* x, int ldx, int T, const float* norm_w, float eps, float* y,
                         int ldy, int accumulate, unsigned* err, fnx_stream st) {
    if (int rc = check_cols(cols)) return rc;
    const int tps = MMV_ITEMS / (cols / 256);
    FNX_REQUIRE(W && x && y && err, "fnx_dense: null pointer");
    FNX_REQUIRE(T >= 1 && T <= 8, "fnx_dense: %d rows per call (1..8)", T);
    FNX_REQUIRE(rows > 0 && rows % (16 * tps) == 0, "fnx_dense: %d output rows, not a multiple of %d for %d columns", rows, 16 * tps, cols);
    FNX_REQUIRE(ldx % 4 == 0 && ((uintptr_t) x & 15) == 0 && ((uintptr_t) W & 15) == 0, "fnx_dense: x and W must be 16-byte aligned");
    MmvParams p{};
    p.W = (const uint8_t*) W;
    p.T = T;
    p.x = x;
    p.ldx = ldx;
    p.norm_w = norm_w;
    p.eps = eps;
    p.out = y;
    p.ldo = ldy;
    p.rows = rows;
    p.K = cols;
    p.accumulate = accumulate;
    p.err = err;
    return T <= 4 ? launch_mmv<1, MMV_DENSE>(p, as_stream(st)) : launch_mmv<2, MMV_DENSE>(p, as_stream(st));
}

extern "C" int fnx_moe_gate_up(const void* Wgu, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs,
                               const int* njobs, int njobs_max, const float* x, const float* norm_w, float eps, int H, int F, float* h,
                               unsigned* err, fnx_stream st) {
    if (int rc = check_cols(H)) return rc;
    const int tps = MMV_ITEMS / (H / 256);
    FNX_REQUIRE(Wgu && jobs && njobs && x && h && err, "fnx_moe_gate_up: null pointer");
    FNX_REQUIRE(tps >= 2 && F % (8 * tps) == 0, "fnx_moe_gate_up: hidden %d, ffn %d not supported", H, F);
    MmvParams p{};
    p.W = (const uint8_t*) Wgu;
    p.expert_stride = expert_stride;
    p.e_base = e_base;
    p.Wsh = (const uint8_t*) Wsh;
    p.E = E;
    p.jobs = jobs;
    p.njobs = njobs;
    p.njobs_max = njobs_max;
    p.x = x;
    p.ldx = H;
    p.norm_w = norm_w;
    p.eps = eps;
    p.out = h;
    p.ldo = F;
    p.rows = F;
    p.K = H;
    p.err = err;
    return launch_mmv<1, MMV_GATEUP>(p, as_stream(st));
}

extern "C" int fnx_moe_down(const void* Wdn, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs, const int* njobs,
                            int njobs_max, const float* h, int H, int F, float* part, unsigned* err, fnx_stream st) {
    if (int rc = check_cols(F)) return rc;
    const int tps = MMV_ITEMS / (F / 256);
    FNX_REQUIRE(Wdn && jobs && njobs && h && part && err, "fnx_moe_down: null pointer");
    FNX_REQUIRE(H % (16 * tps) == 0, "fnx_moe_down: hidden %d not a multiple of %d for ffn %d", H, 16 * tps, F);
    MmvParams p{};
    p.W = (const uint8_t*) Wdn;
    p.expert_stride = expert_stride;
    p.e_base = e_base;
    p.Wsh = (const uint8_t*) Wsh;
    p.E = E;
    p.jobs = jobs;
    p.njobs = njobs;
    p.njobs_max = njobs_max;
    p.x = h;
    p.ldx = F;
    p.out = part;
    p.ldo = H;
    p.rows = H;
    p.K = F;
    p.err = err;
    return launch_mmv<1, MMV_DOWN>(p, as_stream(st));
}
