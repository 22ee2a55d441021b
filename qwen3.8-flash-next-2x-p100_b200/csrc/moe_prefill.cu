// Prefill-sized MoE block: token groups per expert through the 5th-generation tensor cores.
//
// Replaces the reference's grouped expert GEMMs for prompts, moe_gate_up_mma / moe_down_mma
// (engine/src/kernels.hpp:328-330, engine/src/moe_mma.cuh:301) and their job build k_pf_*
// (engine/src/prefill.cu:288-377): the (token, pick) pairs are grouped by expert into jobs of up to 256 rows, and each
// job's product runs as tcgen05.mma (kind::f16, f32 accumulators in tensor memory):
//   A = a 128-feature slab of the expert's IQ3_S matrix, decoded by the block's warps straight from the tile layout
//       (iq3s_tile.h) into f16 in the K-major core-matrix layout the instruction's shared-memory descriptor names;
//   B = the job's activation rows (RMS-normed and rounded to f16 once per call; gathered by 16-byte async copies), same layout;
//   D = [128 features (lanes)] x [256 rows (columns)] in tensor memory; gate|up keeps two of them and the epilogue
//       applies SwiGLU while it reads them back (tcgen05.ld).
// Three shared-memory stages of 64 K columns: the warps decode ahead while the tensor core works on earlier chunks; a stage is reused
// when the tcgen05.commit of its chunk has arrived on the stage's mbarrier.  Every wait is bounded.
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "fnx_common.cuh"
#include "iq3s_grid.h"
#include "iq3s_tile.h"

namespace fnxb {

constexpr int PF_M = 128;         // features per block (tensor-memory lanes)
constexpr int PF_N = 256;         // rows per job (tensor-memory columns per accumulator): a decoded weight slab serves them all
constexpr int PF_KC = 64;         // K per stage: a quarter of a 256-column IQ3_S block (two sub-blocks)
constexpr int PF_THREADS = 512;     // decode threads (16 warps)
constexpr int PF_BLOCK = PF_THREADS + 32;   // + the warp whose lane 0 issues the tensor-core work
constexpr int PF_STAGES = 3;      // operand stages in shared memory: the decode runs up to two chunks ahead of the tensor core
constexpr int PF_REP = 4;          // copies of the codebook (entry e of copy r at word e * 4 + r): lane l reads copy l % 4
// Core matrices (8 rows x 16 bytes = 128 bytes) are laid 144 bytes apart along K: the 16-byte stores of a quarter warp of
// the decode (two rows x four K pieces) then fall into two bank groups per row instead of one (2-way conflicts, not 4-way)
constexpr int PF_LBO = 144;                    // bytes between core matrices along K
constexpr int PF_SBO = (PF_KC / 8) * PF_LBO;   // ... along the rows
constexpr int PF_TILE_A = (PF_M / 8) * PF_SBO; // bytes of one f16 weight tile (128 features x 64)
constexpr int PF_TILE_B = (PF_N / 8) * PF_SBO; // ... of the activation tile (256 rows x 64)

struct PfJob {
    int w, n, start;   // expert, rows, first entry of `order`
};

__device__ static const uint32_t g_grid_pf[512] = {FNX_IQ3S_GRID_VALUES};

// ---- tcgen05 wrappers
__device__ __forceinline__ uint64_t pf_desc(uint32_t saddr) {
    // shared-memory matrix descriptor: start address, leading (K) and stride (row-group) byte offsets in 16-byte units,
    // descriptor version 1, no swizzle
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) (PF_LBO >> 4) << 16) | ((uint64_t) (PF_SBO >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void pf_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pf_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pf_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void pf_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pf_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// byte offset of element (row, k) of a 128 x 128 f16 operand tile in the core-matrix layout
__device__ __forceinline__ uint32_t pf_off(int row, int k) { return (uint32_t) ((row >> 3) * PF_SBO + (k >> 3) * PF_LBO + (row & 7) * 16 + (k & 7) * 2); }

// what a lane holds of one 16 x 256 tile block: the index streams and sign words of rows g and g + 8, their scales
struct PfRaw {
    uint32_t S0[5], S1[5], G0[2], G1[2];
    uint32_t sn0, sn1;
    float d0, d1;
};
__device__ __forceinline__ void pf_load_raw(const uint8_t* tile, int lane, PfRaw& r) {
    const int g = lane >> 2;
    const uint4 i0 = *reinterpret_cast<const uint4*>(tile + TILE_IDX + lane * 16), i1 = *reinterpret_cast<const uint4*>(tile + TILE_IDX + 512 + lane * 16);
    const uint2 s0 = *reinterpret_cast<const uint2*>(tile + TILE_SGN + lane * 8), s1 = *reinterpret_cast<const uint2*>(tile + TILE_SGN + 256 + lane * 8);
    r.S0[0] = i0.x; r.S0[1] = i0.y; r.S0[2] = i0.z; r.S0[3] = i0.w;
    r.S1[0] = i1.x; r.S1[1] = i1.y; r.S1[2] = i1.z; r.S1[3] = i1.w;
    r.S0[4] = *reinterpret_cast<const uint16_t*>(tile + TILE_TAIL + lane * 2);
    r.S1[4] = *reinterpret_cast<const uint16_t*>(tile + TILE_TAIL + 64 + lane * 2);
    r.G0[0] = s0.x; r.G0[1] = s0.y;
    r.G1[0] = s1.x; r.G1[1] = s1.y;
    r.sn0 = *reinterpret_cast<const uint32_t*>(tile + TILE_SCL + g * 4);
    r.sn1 = *reinterpret_cast<const uint32_t*>(tile + TILE_SCL + (g + 8) * 4);
    r.d0 = __half2float(*reinterpret_cast<const __half*>(tile + TILE_D + g * 2));
    r.d1 = __half2float(*reinterpret_cast<const __half*>(tile + TILE_D + (g + 8) * 2));
}

// eight signed codebook bytes (two lookups) times the sub-block scale -> eight f16 at (row, k .. k + 7): one core-matrix
// row.  Bytes become halves without the conversion unit: 0x6400 | (b + 128) is the f16 1024 + (b + 128), exactly.
__device__ __forceinline__ uint4 pf_halves8(uint32_t lo4, uint32_t hi4, __half2 f2) {
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t u = (j < 2 ? lo4 : hi4) ^ 0x80808080u;
        uint32_t pair;
        if (j & 1) asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(pair) : "r"(u), "r"(0x64646464u));
        else asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(pair) : "r"(u), "r"(0x64646464u));
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&pair), bias), f2);
        h[j] = *reinterpret_cast<const uint32_t*>(&v);
    }
    return make_uint4(h[0], h[1], h[2], h[3]);
}
__device__ __forceinline__ void pf_store8(uint8_t* tileA, int row, int k, uint32_t lo4, uint32_t hi4, __half2 f2) {
    *reinterpret_cast<uint4*>(tileA + pf_off(row, k)) = pf_halves8(lo4, hi4, f2);
}

template <int I>
__device__ __forceinline__ uint32_t pf_decode(const uint32_t (&S)[5], const uint32_t (&G)[2], uint32_t table_s) {
    uint32_t mag;
    const uint32_t a = table_s + (tile_field<I>(S) >> 3);   // the field is (index << 7): 16 bytes per entry (PF_REP copies); table_s: the lane's copy
    asm("ld.shared.u32 %0, [%1];" : "=r"(mag) : "r"(a));
    return tile_apply_sign(mag, tile_sign_mask<I>(G));
}

// sub-block SB of the lane's two rows into the operand tile (tile rows row0 + g, row0 + g + 8; columns relative to the
// chunk).  Lane q of a row holds the sub-block's columns 8 q .. 8 q + 7: lookup 2 SB the first four, 2 SB + 1 the others
// (the tile layout pairs them with the activation cells of 8 consecutive columns, iq3s_tile.h).
template <int SB>
__device__ __forceinline__ void pf_sub_block(const PfRaw& r, uint8_t* tileA, int row0, int lane, uint32_t table_s) {
    const int g = lane >> 2, q = lane & 3, k0 = (SB & 1) * 32 + 8 * q;
    const __half2 f0 = __float2half2_rn(r.d0 * (float) (1 + 2 * (int) ((r.sn0 >> (8 * (SB >> 1) + 4 * (SB & 1))) & 15u)));
    const __half2 f1 = __float2half2_rn(r.d1 * (float) (1 + 2 * (int) ((r.sn1 >> (8 * (SB >> 1) + 4 * (SB & 1))) & 15u)));
    pf_store8(tileA, row0 + g, k0, pf_decode<2 * SB>(r.S0, r.G0, table_s), pf_decode<2 * SB + 1>(r.S0, r.G0, table_s), f0);
    pf_store8(tileA, row0 + g + 8, k0, pf_decode<2 * SB>(r.S1, r.G1, table_s), pf_decode<2 * SB + 1>(r.S1, r.G1, table_s), f1);
}
// the warp's share of quarter Q of a tile block (sub-blocks 2 Q, 2 Q + 1): gate|up: both; down (two warps per tile): one
template <int Q, int MODE>
__device__ __forceinline__ void pf_quarter(const PfRaw& r, uint8_t* tileA, int row0, int lane, uint32_t table_s, int sel) {
    if (MODE == 1) {
        pf_sub_block<2 * Q>(r, tileA, row0, lane, table_s);
        pf_sub_block<2 * Q + 1>(r, tileA, row0, lane, table_s);
    } else if (sel == 0) {
        pf_sub_block<2 * Q>(r, tileA, row0, lane, table_s);
    } else {
        pf_sub_block<2 * Q + 1>(r, tileA, row0, lane, table_s);
    }
}

struct PfParams {
    const uint8_t* W;          // experts [e_base ..): gate|up [2 F][K] or down [H][K] tile matrices
    size_t expert_stride;
    int e_base, E;
    const uint8_t* Wsh;        // the shared expert (job.w == E)
    const PfJob* jobs;
    const int* njobs;          // the launch covers the largest possible job count: blocks past *njobs leave at once
    const int* order;          // per job entry: the pair index t * Kp + k; shared jobs: T * Kp + t
    int TKp;                   // T * Kp: entries at or past it are shared-expert rows
    int Kp;
    const __half* x;           // f16 activations: gate|up: [T][K] normed rows (row = token), down: [pairs][K] (row = pair)
    int rows, K;               // output features per expert matrix (gate|up: F; down: H), inner dimension
    float* out;                // down: [pairs][rows] f32
    __half* outh;              // gate|up: [pairs][rows] f16 (the down product's operand)
    unsigned* err;
    int ldo;                   // MODE 0: floats between output rows (0: rows)
    int accumulate;            // MODE 0: out += the product
};

// MODE 0: out = x W^T (down).  MODE 1: out = silu(x Wg^T) * (x Wu^T) (gate|up; W = [gate (rows); up (rows)]).
template <int MODE>
__global__ void __launch_bounds__(PF_BLOCK, 1) k_pf_gemm(const PfParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NA = MODE == 1 ? 2 : 1;                      // weight tiles per stage
    constexpr int STAGE = NA * PF_TILE_A + PF_TILE_B;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* stage0 = smem;                                    // PF_STAGES stages: [A0 | (A1) | B]
    uint32_t* table = reinterpret_cast<uint32_t*>(smem + PF_STAGES * STAGE);          // the codebook, PF_REP copies
    int* src_s = reinterpret_cast<int*>(table + 512 * PF_REP);          // [PF_N] activation row per job row (-1: none)
    int* out_s = src_s + PF_N;                                 // [PF_N] output row
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_s + PF_N);   // [PF_STAGES] stage free (the tensor core's commit)
    uint64_t* full = bars + PF_STAGES;                            // [PF_STAGES] stage filled (one arrival per decode warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(full + PF_STAGES);
    if ((int) blockIdx.x >= *p.njobs) return;   // (before anything is allocated or waited for)
    const PfJob job = p.jobs[blockIdx.x];
    const int ft = blockIdx.y, KB = p.K / 256, nchunk = p.K / PF_KC;
    const uint8_t* W = job.w >= p.E ? p.Wsh : p.W + (size_t) (job.w - p.e_base) * p.expert_stride;
    for (int i = tid; i < 512 * PF_REP; i += PF_BLOCK) table[i] = g_grid_pf[i / PF_REP];
    if (tid < PF_N) {
        int src = -1, o = 0;
        if (tid < job.n) {
            const int pr = p.order[job.start + tid];
            o = pr;
            src = MODE == 1 ? (pr >= p.TKp ? pr - p.TKp : pr / p.Kp) : pr;
        }
        src_s[tid] = src;
        out_s[tid] = o;
    }
    if (tid == 0) {
        for (int i = 0; i < PF_STAGES; ++i) {
            mbar_init(&bars[i], 1);
            mbar_init(&full[i], PF_THREADS / 32);
        }
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NA * PF_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pf_fence_before();
    __syncthreads();
    pf_fence_after();
    const uint32_t tmem = *tmem_slot, table_s = smem_u32(table) + (uint32_t) (lane % PF_REP) * 4u;
    // instruction descriptor: f32 accumulate, f16 x f16, both operands K-major, N = 256, M = 128
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (PF_N >> 3) << 17) | ((uint32_t) (PF_M >> 4) << 24);
    bool ok = true;
    if (warp == PF_THREADS / 32) {
        // the issuing warp: lane 0 waits for a stage to be filled, issues its products, and has their completion free the stage
        if (lane == 0) {
            for (int c = 0; c < nchunk; ++c) {
                const int s = c % PF_STAGES;
                if (!mbar_wait_bounded(&full[s], (unsigned) ((c / PF_STAGES) & 1), 20000000u)) {
                    atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
                    break;
                }
                pf_fence_after();
                const uint32_t a_s = smem_u32(stage0 + (size_t) s * STAGE), b_s = a_s + NA * PF_TILE_A;
#pragma unroll
                for (int k16 = 0; k16 < PF_KC / 16; ++k16) {
                    const uint64_t bd = pf_desc(b_s + k16 * 2 * PF_LBO);
                    pf_mma(tmem, pf_desc(a_s + k16 * 2 * PF_LBO), bd, IDESC, (c | k16) != 0);
                    if (NA == 2) pf_mma(tmem + PF_N, pf_desc(a_s + PF_TILE_A + k16 * 2 * PF_LBO), bd, IDESC, (c | k16) != 0);
                }
                pf_commit(&bars[s]);
            }
        }
        __syncwarp();
    } else {
        // 16 warps: warp w decodes tile row (w % 8) of the 128-feature slab; gate|up: of the gate (w < 8) or the up matrix
        // (all four sub-blocks of the chunk); down: sub-block pair w / 8 of the chunk
        PfRaw raw, nxt;
        const int sel = warp >> 3;
        const int trow = (MODE == 1 && sel ? p.rows / 16 : 0) + ft * (PF_M / 16) + (warp & 7);
        const int a_off = MODE == 1 && sel ? PF_TILE_A : 0, row0 = (warp & 7) * 16;
        // (a slab past the matrix's last tile row, when the features are not a multiple of 128, decodes zero weights)
        const bool live_row = MODE == 1 || trow < p.rows / 16;
        auto load_raw = [&](int kb, PfRaw& r) {
            if (live_row) pf_load_raw(W + ((size_t) trow * KB + kb) * TILE_BYTES, lane, r);
            else r = PfRaw{};
        };
        load_raw(0, raw);
        // the activations of chunk c into its stage: 16-byte pieces (8 columns of one row = one core-matrix row) by async copies;
        // they run one chunk ahead of the decode, so their latency hides behind it
        auto issue_b = [&](int c) {
            uint8_t* B = stage0 + (size_t) (c % PF_STAGES) * STAGE + NA * PF_TILE_A;
#pragma unroll
            for (int j = 0; j < PF_N * (PF_KC / 8) / PF_THREADS; ++j) {
                // consecutive lanes take consecutive rows of one 8-column piece: the eight 16-byte stores of a quarter warp fill one
                // 128-byte core matrix (no bank conflicts); the global side reads half sectors, which the L2 absorbs
                const int i = tid + j * PF_THREADS, brow = i & (PF_N - 1), piece = i / PF_N;
                const int src = src_s[brow];
                uint8_t* dst = B + pf_off(brow, piece * 8);
                if (src >= 0) {
                    const __half* g = p.x + (size_t) src * p.K + c * PF_KC + piece * 8;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(g) : "memory");
                } else {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                }
            }
        };
        issue_b(0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        for (int c = 0; c < nchunk; ++c) {
            const int s = c % PF_STAGES, kb = c >> 2, quarter = c & 3;
            uint8_t* A0 = stage0 + (size_t) s * STAGE;
            bool gave_up = false;
            if (c + 1 < nchunk) {
                // the next chunk's stage is free when the tensor core has finished the chunk that used it (a wait that gives up is
                // reported at the chunk's one block barrier below, where every thread takes the same exit)
                if (c + 1 >= PF_STAGES) {
                    gave_up = !mbar_wait_bounded(&bars[(c + 1) % PF_STAGES], (unsigned) (((c + 1) / PF_STAGES - 1) & 1), 20000000u);
                    pf_fence_after();
                }
                issue_b(c + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            // the weights of this chunk: four sub-blocks of the warp's tile(s); the next block's bytes are fetched meanwhile
            switch (quarter) {
                case 0:
                    pf_quarter<0, MODE>(raw, A0 + a_off, row0, lane, table_s, sel);
                    if (kb + 1 < KB) load_raw(kb + 1, nxt);
                    break;
                case 1: pf_quarter<1, MODE>(raw, A0 + a_off, row0, lane, table_s, sel); break;
                case 2: pf_quarter<2, MODE>(raw, A0 + a_off, row0, lane, table_s, sel); break;
                default:
                    pf_quarter<3, MODE>(raw, A0 + a_off, row0, lane, table_s, sel);
                    raw = nxt;
                    break;
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");   // this chunk's activations are in; the next chunk's may still fly
            fence_proxy_async();   // the tiles were written through the generic proxy; the tensor core reads them through the async one
            if (__any_sync(0xffffffffu, gave_up)) {   // no arrival: the issuing warp's wait runs out and reports it
                ok = false;
                break;
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[s])) : "memory");
        }
    }
    // all chunks issued: the last commit arrives when every earlier product has finished too
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // every warp takes this barrier, whatever it saw: a warp that gave up votes "not ok" without waiting, and the block agrees on one
    // answer before anything reads or frees the accumulators
    ok = __syncthreads_and(ok && mbar_wait_bounded(&bars[(nchunk - 1) % PF_STAGES], (unsigned) (((nchunk - 1) / PF_STAGES) & 1), 20000000u)) != 0;
    pf_fence_after();
    if (!ok && tid == 0) atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
    if (ok && warp < PF_THREADS / 32) {
        // warp w reads lanes 32 (w % 4) .. + 31 (its features), columns 64 (w / 4) .. + 63 (job rows), 32 at a time
        const int f = ft * PF_M + 32 * (warp & 3) + lane;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            const int col0 = (warp >> 2) * 64 + hh * 32;
            if (col0 >= job.n) break;
            const uint32_t ta = tmem + ((uint32_t) (32 * (warp & 3)) << 16) + (uint32_t) col0;
            float g[32];
            pf_ld32(ta, g);
            if (MODE == 1) {
                float u[32];
                pf_ld32(ta + PF_N, u);
#pragma unroll
                for (int i = 0; i < 32; ++i) g[i] = siluf_(g[i]) * u[i];
            }
            const int ldo = MODE == 0 && p.ldo ? p.ldo : p.rows;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col0 + i < job.n && f < p.rows) {
                    if (MODE == 1) p.outh[(size_t) out_s[col0 + i] * p.rows + f] = __float2half_rn(g[i]);
                    else {
                        float* o = p.out + (size_t) out_s[col0 + i] * ldo + f;
                        *o = p.accumulate ? *o + g[i] : g[i];
                    }
                }
        }
    }
    pf_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NA * PF_N) : "memory");
}

// ------------------------------------------------------------------------------------------------ job build
// per expert: how many pairs picked it
__global__ void k_pf_count(const int* __restrict__ topi, int n, int e_lo, int* __restrict__ cnt) {
    const int e = e_lo + blockIdx.x;
    int c = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) c += topi[i] == e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    __shared__ int ws[32];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int w = 0; w < (int) blockDim.x / 32; ++w) s += ws[w];
        cnt[blockIdx.x] = s;
    }
}

// one block: the experts' first entries and jobs (ascending expert order, then the shared expert's)
__global__ void k_pf_plan(const int* __restrict__ cnt, int ne, int e_lo, int E, int T, int TKp, int add_shared, int* __restrict__ base, PfJob* __restrict__ jobs,
                          int* __restrict__ njobs, int* __restrict__ order) {
    // counts into shared memory, one thread's running sums over them (a few hundred shared-memory steps), then every thread
    // writes its experts' jobs
    __shared__ int s_cnt[1024], s_entry[1024], s_job[1024];
    __shared__ int s_entries, s_jobs;
    for (int e = threadIdx.x; e < ne; e += blockDim.x) s_cnt[e] = cnt[e];
    __syncthreads();
    if (threadIdx.x == 0) {
        int entry = 0, nj = 0;
        for (int e = 0; e < ne; ++e) {
            s_entry[e] = entry;
            s_job[e] = nj;
            entry += s_cnt[e];
            nj += (s_cnt[e] + PF_N - 1) / PF_N;
        }
        s_entries = entry;
        s_jobs = nj;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < ne; e += blockDim.x) {
        base[e] = s_entry[e];
        int j = s_job[e];
        for (int o = 0; o < s_cnt[e]; o += PF_N) jobs[j++] = PfJob{e_lo + e, min(PF_N, s_cnt[e] - o), s_entry[e] + o};
    }
    const int entry = s_entries, nj = s_jobs;
    if (add_shared) {
        for (int t = threadIdx.x; t < T; t += blockDim.x) order[entry + t] = TKp + t;
        for (int j = threadIdx.x; j < (T + PF_N - 1) / PF_N; j += blockDim.x) jobs[nj + j] = PfJob{E, min(PF_N, T - j * PF_N), entry + j * PF_N};
    }
    if (threadIdx.x == 0) njobs[0] = nj + (add_shared ? (T + PF_N - 1) / PF_N : 0);
}

// per expert: its pairs in ascending order into order[base ..): a thread looks at four consecutive pairs per step
__global__ void k_pf_fill(const int* __restrict__ topi, int n, int e_lo, const int* __restrict__ base, int* __restrict__ order) {
    const int e = e_lo + blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x / 32;
    __shared__ int ws[32], s_run;
    if (tid == 0) s_run = base[blockIdx.x];
    __syncthreads();
    const bool vec = (((uintptr_t) topi) & 15) == 0;
    for (int i0 = 0; i0 < n; i0 += blockDim.x * 4) {
        const int i = i0 + tid * 4;
        int v[4] = {-1, -1, -1, -1};
        if (vec && i + 3 < n) {
            const int4 q = *reinterpret_cast<const int4*>(topi + i);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + j < n) v[j] = topi[i + j];
        }
        int c = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) c += v[j] == e;
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += u;
        }
        if (lane == 31) ws[warp] = incl;
        __syncthreads();
        int before = incl - c, total = 0;
        for (int w = 0; w < nw; ++w) {
            if (w < warp) before += ws[w];
            total += ws[w];
        }
        const int run = s_run;
        int at = run + before;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (v[j] == e) order[at++] = i + j;
        __syncthreads();
        if (tid == 0) s_run = run + total;
        __syncthreads();
    }
}

// xh[t] = f16(x[t] * norm_w / rms(x[t]))   (norm_w null: f16(x[t]))
__global__ void k_pf_xnorm(const float* __restrict__ x, const float* __restrict__ norm_w, int H, float eps, __half* __restrict__ xh) {
    const float* xr = x + (size_t) blockIdx.x * H;
    __shared__ float ws[32], s_r;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int) blockDim.x / 32; ++w) t += ws[w];
        s_r = norm_w ? rsqrtf(t / (float) H + eps) : 1.0f;
    }
    __syncthreads();
    const float r = s_r;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(xr + i);
        if (norm_w) {
            const float4 w = *reinterpret_cast<const float4*>(norm_w + i);
            v.x *= w.x * r; v.y *= w.y * r; v.z *= w.z * r; v.w *= w.w * r;
        }
        const __half2 a = __floats2half2_rn(v.x, v.y), b2 = __floats2half2_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(xh + (size_t) blockIdx.x * H + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b2));
    }
}

// out[t] (+)= sum_k topw[t][k] part[t Kp + k] + sigmoid(logit[t][E]) part[T Kp + t]
__global__ void k_pf_combine(const float* __restrict__ part, const int* __restrict__ topi, const float* __restrict__ topw, const float* __restrict__ logits,
                             int T, int E, int H, int Kp, int e_lo, int e_hi, int add_shared, float* __restrict__ out, int accumulate) {
    // a thread owns four columns of one row; the picks' weights first, then every addend's 16-byte load in flight at once
    const int t = blockIdx.y, i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= H) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < Kp; k0 += 16) {   // sixteen picks at a time (the sum stays in pick order)
        float w[16];
        float4 v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            w[k] = 0.f;
            if (k0 + k < Kp) {
                const int e = topi[t * Kp + k0 + k];
                w[k] = e >= e_lo && e < e_hi ? topw[t * Kp + k0 + k] : 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < 16; ++k)
            v[k] = w[k] != 0.f ? *reinterpret_cast<const float4*>(part + ((size_t) t * Kp + k0 + k) * H + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            s.x = fmaf(w[k], v[k].x, s.x); s.y = fmaf(w[k], v[k].y, s.y);
            s.z = fmaf(w[k], v[k].z, s.z); s.w = fmaf(w[k], v[k].w, s.w);
        }
    }
    if (add_shared) {
        const float g = sigmoidf_(logits[(size_t) t * (E + 1) + E]);
        const float4 sh = *reinterpret_cast<const float4*>(part + ((size_t) T * Kp + t) * H + i);
        s.x += g * sh.x; s.y += g * sh.y; s.z += g * sh.z; s.w += g * sh.w;
    }
    float4* o = reinterpret_cast<float4*>(out + (size_t) t * H + i);
    if (accumulate) {
        const float4 p0 = *o;
        s.x += p0.x; s.y += p0.y; s.z += p0.z; s.w += p0.w;
    }
    *o = s;
}

// A tile matrix decoded once to f16, row-major [rows][K]: the values the grouped product's own decode makes (the same codebook
// bytes, scales and half arithmetic), for the products that take their weights by tensor copies (gemm_tma.cu).  One warp per
// 16 x 256 tile block.
__global__ void __launch_bounds__(256) k_pf_decode_f16(const uint8_t* __restrict__ W, int rows, int K, __half* __restrict__ out) {
    __shared__ uint32_t table[512 * PF_REP];
    for (int i = threadIdx.x; i < 512 * PF_REP; i += blockDim.x) table[i] = g_grid_pf[i / PF_REP];
    __syncthreads();
    const int lane = threadIdx.x & 31, KB = K / 256;
    const size_t nblk = (size_t) (rows / 16) * KB;
    const uint32_t table_s = smem_u32(table) + (uint32_t) (lane % PF_REP) * 4u;
    const int g = lane >> 2, q = lane & 3;
    for (size_t b = (size_t) blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5); b < nblk; b += (size_t) gridDim.x * (blockDim.x / 32)) {
        const size_t trow = b / KB;
        const int kb = (int) (b % KB);
        PfRaw r;
        pf_load_raw(W + b * TILE_BYTES, lane, r);
        __half* o0 = out + (trow * 16 + g) * K + (size_t) kb * 256 + 8 * q;
        __half* o1 = o0 + (size_t) 8 * K;
        auto sub = [&](auto SBc) {
            constexpr int SB = decltype(SBc)::value;
            const __half2 f0 = __float2half2_rn(r.d0 * (float) (1 + 2 * (int) ((r.sn0 >> (8 * (SB >> 1) + 4 * (SB & 1))) & 15u)));
            const __half2 f1 = __float2half2_rn(r.d1 * (float) (1 + 2 * (int) ((r.sn1 >> (8 * (SB >> 1) + 4 * (SB & 1))) & 15u)));
            *reinterpret_cast<uint4*>(o0 + SB * 32) = pf_halves8(pf_decode<2 * SB>(r.S0, r.G0, table_s), pf_decode<2 * SB + 1>(r.S0, r.G0, table_s), f0);
            *reinterpret_cast<uint4*>(o1 + SB * 32) = pf_halves8(pf_decode<2 * SB>(r.S1, r.G1, table_s), pf_decode<2 * SB + 1>(r.S1, r.G1, table_s), f1);
        };
        sub(std::integral_constant<int, 0>{}); sub(std::integral_constant<int, 1>{}); sub(std::integral_constant<int, 2>{}); sub(std::integral_constant<int, 3>{});
        sub(std::integral_constant<int, 4>{}); sub(std::integral_constant<int, 5>{}); sub(std::integral_constant<int, 6>{}); sub(std::integral_constant<int, 7>{});
    }
}

int pf_decode_f16_launch(const void* W, int rows, int K, __half* out, cudaStream_t st) {
    const size_t nblk = (size_t) (rows / 16) * (K / 256);
    const unsigned blocks = (unsigned) (nblk / 8 < 148 * 8 ? (nblk + 7) / 8 : 148 * 8);
    k_pf_decode_f16<<<blocks, 256, 0, st>>>((const uint8_t*) W, rows, K, out);
    FNX_LAUNCH_OK("k_pf_decode_f16");
    return FNX_OK;
}

// the job list of a dense product over T rows: job j = rows [256 j, 256 j + 256) of "expert" 0, entries in row order
__global__ void k_pf_dense_jobs(int T, PfJob* __restrict__ jobs, int* __restrict__ njobs, int* __restrict__ order) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x, nj = (T + PF_N - 1) / PF_N;
    if (i < T) order[i] = i;
    if (i < nj) jobs[i] = PfJob{0, min(PF_N, T - i * PF_N), i * PF_N};
    if (i == 0) *njobs = nj;
}

constexpr size_t pf_smem(int mode) { return (size_t) PF_STAGES * ((mode == 1 ? 2 : 1) * PF_TILE_A + PF_TILE_B) + 2048 * PF_REP + 2 * PF_N * sizeof(int) + 64; }

}  // namespace fnxb

using namespace fnxb;

static size_t pf_align(size_t v) { return (v + 255) & ~(size_t) 255; }

// the rows of the job list's entries, in entry order: x_sorted[pos] = xh[token of order[pos]] (a routed pair t K + k: token t; a
// shared-expert entry n + t: token t), so that a job's rows are consecutive for the tensor copies
__global__ void __launch_bounds__(256) k_pf_gather_rows(const __half* __restrict__ xh, const int* __restrict__ order, int n, int Kp, int H, __half* __restrict__ xs) {
    const int pos = blockIdx.x, pair = order[pos], t = pair < n ? pair / Kp : pair - n;
    const uint4* src = reinterpret_cast<const uint4*>(xh + (size_t) t * H);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t) pos * H);
    for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = src[i];
}

namespace fnxb {
int gemm_tma_experts(const __half* gu16, const __half* dn16, int slots, const __half* x_sorted, __half* h_sorted, float* part, const void* jobs, const int* njobs,
                     const int* order, int max_jobs, int entries, int H, int F, unsigned* err, cudaStream_t st);
static bool pf_gemm_off() {
    static const bool v = []() { const char* e = getenv("FNX_PROMPT_GEMM"); return e && atoi(e) == 0; }();
    return v;
}
// bytes of the f16 copies the tensor-copy form of the experts keeps: the rows in job order, every expert's two matrices
static size_t pf_staged_bytes(size_t pairs, int E, int H, int F) {
    return pf_align(pairs * H * sizeof(__half)) + pf_align((size_t) (E + 1) * 2 * F * H * sizeof(__half)) + pf_align((size_t) (E + 1) * H * F * sizeof(__half));
}
}  // namespace fnxb

extern "C" size_t fnx_moe_prefill_scratch_bytes(int T, int K, int E, int H, int F) {
    const size_t pairs = (size_t) T * K + T;
    return pf_align(pairs * F * sizeof(__half)) + pf_align(pairs * H * sizeof(float)) + pf_align(pairs * sizeof(int)) + pf_align((size_t) (E + 1) * sizeof(int)) * 2 +
           pf_align((pairs / PF_N + E + 2 + (size_t) T / PF_N) * sizeof(PfJob)) + pf_align((size_t) T * H * sizeof(__half)) + 256 +
           (T >= 1024 ? pf_staged_bytes(pairs, E, H, F) : 0);
}

extern "C" int fnx_moe_prefill(const void* Wgu, size_t gu_stride, const void* Wdn, size_t dn_stride, const void* Wsh_gu, const void* Wsh_dn, int e_base,
                               int E, int K, int e_lo, int e_hi, int add_shared, const int* topi, const float* topw, const float* logits, const float* x,
                               const float* norm_w, float eps, int T, int H, int F, float* out, int accumulate, void* scratch, unsigned* err, fnx_stream st_) {
    FNX_REQUIRE(Wgu && Wdn && topi && topw && logits && x && out && scratch && err, "fnx_moe_prefill: null pointer");
    FNX_REQUIRE(T >= 1 && K >= 1 && K <= 32, "fnx_moe_prefill: %d rows, top %d", T, K);
    FNX_REQUIRE(E >= 1 && E <= 1024, "fnx_moe_prefill: %d experts (at most 1024)", E);
    FNX_REQUIRE(H % 256 == 0 && F % 256 == 0 && F % PF_M == 0 && H % PF_M == 0, "fnx_moe_prefill: hidden %d, ffn %d (multiples of 256)", H, F);
    FNX_REQUIRE(0 <= e_lo && e_lo <= e_hi && e_hi <= E && (!add_shared || (Wsh_gu && Wsh_dn)), "fnx_moe_prefill: expert range [%d, %d) of %d", e_lo, e_hi, E);
    FNX_REQUIRE((long long) T * K + T < (1ll << 30), "fnx_moe_prefill: %d rows are too many", T);
    cudaStream_t st = as_stream(st_);
    const size_t pairs = (size_t) T * K + T;
    uint8_t* b = (uint8_t*) scratch;
    __half* hbuf = (__half*) b; b += pf_align(pairs * F * sizeof(__half));
    float* part = (float*) b; b += pf_align(pairs * H * sizeof(float));
    int* order = (int*) b; b += pf_align(pairs * sizeof(int));
    int* cnt = (int*) b; b += pf_align((size_t) (E + 1) * sizeof(int));
    int* base = (int*) b; b += pf_align((size_t) (E + 1) * sizeof(int));
    PfJob* jobs = (PfJob*) b; b += pf_align((pairs / PF_N + E + 2 + (size_t) T / PF_N) * sizeof(PfJob));
    __half* xh = (__half*) b; b += pf_align((size_t) T * H * sizeof(__half));
    int* njobs = (int*) b; b += 256;
    const int ne = e_hi - e_lo, n = T * K;
    if (ne > 0) {
        k_pf_count<<<ne, 1024, 0, st>>>(topi, n, e_lo, cnt);
        FNX_LAUNCH_OK("k_pf_count");
    }
    k_pf_plan<<<1, 256, 0, st>>>(cnt, ne, e_lo, E, T, n, add_shared, base, jobs, njobs, order);
    FNX_LAUNCH_OK("k_pf_plan");
    if (ne > 0) {
        k_pf_fill<<<ne, 256, 0, st>>>(topi, n, e_lo, base, order);
        FNX_LAUNCH_OK("k_pf_fill");
    }
    k_pf_xnorm<<<T, 256, 0, st>>>(x, norm_w, H, eps, xh);
    FNX_LAUNCH_OK("k_pf_xnorm");
    // From 1,024 rows on, with every expert on this rank and stacked without gaps: the experts' matrices decoded to f16 once, the
    // rows copied into job order, and the two grouped products with both operands by tensor copies (gemm_tma.cu).
    if (T >= 1024 && !pf_gemm_off() && e_base == 0 && e_lo == 0 && e_hi == E && add_shared && gu_stride == fnx_iq3s_bytes((size_t) 2 * F, (size_t) H) &&
        dn_stride == fnx_iq3s_bytes((size_t) H, (size_t) F)) {
        __half* xs = (__half*) b; b += pf_align(pairs * H * sizeof(__half));
        __half* gu16 = (__half*) b; b += pf_align((size_t) (E + 1) * 2 * F * H * sizeof(__half));
        __half* dn16 = (__half*) b;
        FNX_TRY(pf_decode_f16_launch(Wgu, E * 2 * F, H, gu16, st));
        FNX_TRY(pf_decode_f16_launch(Wsh_gu, 2 * F, H, gu16 + (size_t) E * 2 * F * H, st));
        FNX_TRY(pf_decode_f16_launch(Wdn, E * H, F, dn16, st));
        FNX_TRY(pf_decode_f16_launch(Wsh_dn, H, F, dn16 + (size_t) E * H * F, st));
        k_pf_gather_rows<<<(unsigned) pairs, 256, 0, st>>>(xh, order, n, K, H, xs);
        FNX_LAUNCH_OK("k_pf_gather_rows");
        const int nj = (int) ((size_t) n / PF_N) + ne + (T + PF_N - 1) / PF_N;
        FNX_TRY(gemm_tma_experts(gu16, dn16, E + 1, xs, hbuf, part, jobs, njobs, order, nj, (int) pairs, H, F, err, st));
        k_pf_combine<<<dim3((H / 4 + 255) / 256, T), 256, 0, st>>>(part, topi, topw, logits, T, E, H, K, e_lo, e_hi, add_shared, out, accumulate);
        FNX_LAUNCH_OK("k_pf_combine");
        return FNX_OK;
    }
    if (int rc = set_smem_limit((const void*) k_pf_gemm<0>, (int) pf_smem(0))) return rc;
    if (int rc = set_smem_limit((const void*) k_pf_gemm<1>, (int) pf_smem(1))) return rc;
    // the job count is known on the device only: the grids cover the largest it can be (an expert's pairs in jobs of PF_N rows:
    // at most one ragged job per expert beyond pairs / PF_N) and the blocks past the count leave at once; nothing is read back
    {
        const int nj = (int) ((size_t) n / PF_N) + ne + (add_shared ? (T + PF_N - 1) / PF_N : 0);
        PfParams p{};
        p.W = (const uint8_t*) Wgu; p.expert_stride = gu_stride; p.e_base = e_base; p.E = E; p.Wsh = (const uint8_t*) Wsh_gu;
        p.jobs = jobs; p.njobs = njobs; p.order = order; p.TKp = n; p.Kp = K; p.x = xh; p.rows = F; p.K = H; p.outh = hbuf; p.err = err;
        k_pf_gemm<1><<<dim3(nj, F / PF_M), PF_BLOCK, pf_smem(1), st>>>(p);
        FNX_LAUNCH_OK("k_pf_gemm (gate|up)");
        p.W = (const uint8_t*) Wdn; p.expert_stride = dn_stride; p.Wsh = (const uint8_t*) Wsh_dn;
        p.x = hbuf; p.rows = H; p.K = F; p.out = part; p.outh = nullptr;
        k_pf_gemm<0><<<dim3(nj, H / PF_M), PF_BLOCK, pf_smem(0), st>>>(p);
        FNX_LAUNCH_OK("k_pf_gemm (down)");
    }
    k_pf_combine<<<dim3((H / 4 + 255) / 256, T), 256, 0, st>>>(part, topi, topw, logits, T, E, H, K, e_lo, e_hi, add_shared, out, accumulate);
    FNX_LAUNCH_OK("k_pf_combine");
    return FNX_OK;
}

// ------------------------------------------------------------------------------------------------ dense product for prompts
namespace fnxb {
int gemm_tma_launch(const __half* w, const __half* wl, const __half* x, const __half* xl, float* y, int ldy, int T, int rows, int K, int accumulate, float scale,
                    unsigned* err, cudaStream_t st);
// rows from which the product takes its weights decoded to f16 once (k_pf_decode_f16) and both operands by tensor copies
// (gemm_tma.cu); FNX_PROMPT_GEMM=0 keeps every product on the form that decodes inside the product
static int pf_tma_rows() {
    static const int v = []() { const char* e = getenv("FNX_PROMPT_GEMM"); return e && atoi(e) == 0 ? 1 << 30 : 1024; }();
    return v;
}
}  // namespace fnxb

extern "C" size_t fnx_dense_prompt_scratch_bytes(int T, int rows, int cols) {
    return pf_align((size_t) T * cols * sizeof(__half)) + pf_align((size_t) T * sizeof(int)) + pf_align(((size_t) T / PF_N + 2) * sizeof(PfJob)) + 256 +
           pf_align((size_t) rows * cols * sizeof(__half));
}

extern "C" int fnx_dense_prompt(const void* W, int rows, int cols, const float* x, int T, const float* norm_w, float eps, float* y, int ldy, int accumulate,
                                void* scratch, unsigned* err, fnx_stream st_) {
    FNX_REQUIRE(W && x && y && scratch && err, "fnx_dense_prompt: null pointer");
    FNX_REQUIRE(T >= 1 && rows >= 16 && rows % 16 == 0 && cols >= 256 && cols % 256 == 0 && ldy >= rows, "fnx_dense_prompt: %d rows x %d columns over %d rows", rows, cols, T);
    cudaStream_t st = as_stream(st_);
    uint8_t* b = (uint8_t*) scratch;
    __half* xh = (__half*) b; b += pf_align((size_t) T * cols * sizeof(__half));
    int* order = (int*) b; b += pf_align((size_t) T * sizeof(int));
    PfJob* jobs = (PfJob*) b; b += pf_align(((size_t) T / PF_N + 2) * sizeof(PfJob));
    int* njobs = (int*) b; b += 256;
    __half* w16 = (__half*) b;
    const int nj = (T + PF_N - 1) / PF_N;
    k_pf_xnorm<<<T, 256, 0, st>>>(x, norm_w, cols, eps, xh);
    FNX_LAUNCH_OK("k_pf_xnorm");
    if (T >= pf_tma_rows()) {   // the matrix to f16 once, then one product with both operands by tensor copies
        FNX_TRY(pf_decode_f16_launch(W, rows, cols, w16, st));
        return gemm_tma_launch(w16, nullptr, xh, nullptr, y, ldy, T, rows, cols, accumulate, 1.0f, err, st);
    }
    k_pf_dense_jobs<<<(T + 255) / 256, 256, 0, st>>>(T, jobs, njobs, order);
    FNX_LAUNCH_OK("k_pf_dense_jobs");
    if (int rc = set_smem_limit((const void*) k_pf_gemm<0>, (int) pf_smem(0))) return rc;
    PfParams p{};
    p.W = (const uint8_t*) W; p.expert_stride = 0; p.e_base = 0; p.E = 1; p.Wsh = nullptr;
    p.jobs = jobs; p.njobs = njobs; p.order = order; p.TKp = T; p.Kp = 1; p.x = xh; p.rows = rows; p.K = cols; p.out = y; p.outh = nullptr; p.err = err;
    p.ldo = ldy; p.accumulate = accumulate;
    k_pf_gemm<0><<<dim3(nj, (rows + PF_M - 1) / PF_M), PF_BLOCK, pf_smem(0), st>>>(p);
    FNX_LAUNCH_OK("k_pf_gemm (dense)");
    return FNX_OK;
}
