// One matrix stage of a block: the body of the IQ3_S matrix x rows kernel (iq3s_mmv.cu).  The block quantises the
// activation rows it needs into its own shared-memory images (or copies the image their producer left), streams its share of the tile blocks through the warps' rings (mmv_core.cuh), combines
// the pieces of tiles cut by warp shares, and writes the results.
#pragma once

#include "mmv_core.cuh"

namespace fnxb {

constexpr int MMV_THREADS = 512, MMV_WARPS = 16;

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
    int R;      // ring slots per warp
    unsigned* err;
    // dense: the rows' image, already built (stage_image_bytes() bytes in the layout of the block's own image): the
    // block copies it instead of quantising x
    const uint8_t* ximg;
};

// bytes of a dense image of NG row groups over K columns: cells, scales, block sums of squares (the order the block
// holds them in)
__host__ __device__ inline size_t stage_image_bytes(int NG, int K) {
    return (size_t) NG * ((size_t) (K / 32) * 32 * 8 + (size_t) (K / 256) * 8 * 4 + 4 * 16 * 4);
}

// jobs whose activation images a block holds at once: its range of units spans at most two jobs of gate|up and a
// few of down; anything wider is walked in passes
template <int MODE>
__host__ __device__ constexpr int mmv_jmax() { return MODE == MAT_DENSE ? 1 : MODE == MAT_GATEUP ? 2 : 4; }

template <int NG, int MODE>
__host__ __device__ inline size_t mmv_image_bytes(int K) {
    return (size_t) mmv_jmax<MODE>() * NG * ((size_t) (K / 32) * 32 * 8 + (size_t) (K / 256) * 8 * 4);
}
template <int NG, int MODE>
__host__ __device__ inline size_t mmv_smem_bytes(int K, int R, int njobs_max) {
    constexpr int rows = mmv_jmax<MODE>() * 4 * NG;
    return (size_t) CORE_TABLE_BYTES + (size_t) MMV_WARPS * R * (TILE_BYTES + 8) + mmv_image_bytes<NG, MODE>(K) + rows * 16 * sizeof(float) +
           (size_t) MMV_WARPS * 2 * sizeof(PieceSlotT<NG, MODE>) + (MODE == MAT_DENSE ? 0 : (size_t) njobs_max * sizeof(fnx_job)) + 64;
}

constexpr int MMV_JOB_WORDS = sizeof(fnx_job) / 4, MMV_JOB_REGS = 3;   // job-list words a thread holds across the set-up

// the block's shared memory for a stage (carved by the caller; the table is filled and the barriers initialised)
struct StageSmem {
    uint32_t table_s;       // the replicated codebook
    uint8_t* slots;         // MMV_WARPS x R tile-block slots
    uint64_t* bars;         // MMV_WARPS x bar_stride mbarriers (they live as long as the kernel)
    int bar_stride;
    uint2* cells;           // images: jmax x NG x (K / 32) x 32 cells, then their scales and chunk sums
    float* scales;
    float* rs;
    void* pieces;           // MMV_WARPS x 2 piece slots (PieceSlotT of the stage's row groups and mode)
    fnx_job* jobs_s;        // njobs_max jobs (expert modes)
};

// what a thread holds from stage_begin() to stage_run(): loads in flight
struct StageRegs {
    int njobs;
    int jw[MMV_JOB_REGS];
    float v[QUANT_BATCH][8];
    float w[QUANT_BATCH][8];   // their norm weights
};

// no-op transform of a fetched block (row t, block blk: 8 values per lane)
struct RowPlain {
    __device__ __forceinline__ void operator()(int, int, int, float (&)[8]) const {}
};

// dense stage: task id -> (row id % T, block id / T)
__device__ __forceinline__ QuantTask stage_dense_task(const MmvParams& p, int id) {
    QuantTask q;
    q.src = nullptr;
    q.t = q.blk = 0;
    if (id < p.T * (p.K / 256)) {
        q.t = id % p.T;
        q.blk = id / p.T;
        q.src = p.x + (size_t) q.t * p.ldx + q.blk * 256;
    }
    return q;
}

// points the warp's (empty) ring at its slots for a stage of depth R
__device__ __forceinline__ void stage_ring(WarpRing& ring, const StageSmem& S, int R, int warp) {
    ring.slots = S.slots + (size_t) warp * R * TILE_BYTES;
    ring.slots_s = smem_u32(ring.slots);
    ring.bars = S.bars + warp * S.bar_stride;
    ring_reset(ring, R);
}

// Starts the loads whose latency the caller may hide behind other work: the job list (expert modes) or the warp's
// first rows to quantise (dense).  post(t, chunk, lane, v) may transform a fetched dense chunk of row t in place.
template <int NG, int MODE, int NW = MMV_WARPS, typename Post>
__device__ __forceinline__ void stage_begin(const MmvParams& p, StageRegs& h, int tid, Post&& post) {
    constexpr bool MOE = MODE != MAT_DENSE;
    constexpr int NROW = mmv_jmax<MODE>() * 4 * NG;
    const int warp = tid >> 5, lane = tid & 31;
    h.njobs = 1;
    if (MOE) {
        const int nword = p.njobs_max * MMV_JOB_WORDS;
        h.njobs = *p.njobs;
#pragma unroll
        for (int i = 0; i < MMV_JOB_REGS; ++i) {
            const int w = tid + i * (NW * 32);
            h.jw[i] = w < nword ? reinterpret_cast<const int*>(p.jobs)[w] : 0;
        }
    } else if (p.ximg) {
        // the image's first 16-byte words ride in the registers the rows would have used
        static_assert(QUANT_BATCH == 2, "eight 16-byte words per thread");
        const int n16 = (int) (stage_image_bytes(NG, p.K) / 16);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = tid + j * (NW * 32);
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n16) t = __ldcg(reinterpret_cast<const float4*>(p.ximg) + i);
            float* d = j < 4 ? &h.v[j >> 1][(j & 1) * 4] : &h.w[(j - 4) >> 1][(j & 1) * 4];
            d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < QUANT_BATCH; ++j) {
            const QuantTask q = stage_dense_task(p, warp + j * NW);
            quant_fetch(q, p.norm_w, lane, h.v[j], h.w[j]);
            if (q.src) post(q.t, q.blk, lane, h.v[j]);
        }
    }
}

// The stage proper.  `bid` of `nblk` blocks of NW warps share the matrix.  ring: the warp's ring, empty, set by stage_ring() (with
// ring.pre set when mat_preissue() already ran for this block's first pass: dense stages only, whose weights do not
// depend on what the stage waits for).  Ends with every result of the block written (no trailing barrier).
// stamp(): a tracing hook called at the phase boundaries.
template <int NG, int MODE, int NW = MMV_WARPS, typename Post, typename Stamp>
__device__ __forceinline__ void stage_run(const MmvParams& p, const StageSmem& S, WarpRing& ring, StageRegs& h, int tid, int bid, int nblk, Post&& post,
                                          Stamp&& stamp) {
    constexpr int JMAX = mmv_jmax<MODE>(), NROW = JMAX * 4 * NG;
    constexpr bool MOE = MODE != MAT_DENSE;
    const int warp = tid >> 5, lane = tid & 31;
    const int KB = p.K / 256;
    int njobs = 1;
    if (MOE) {
        const int nword = p.njobs_max * MMV_JOB_WORDS;
#pragma unroll
        for (int i = 0; i < MMV_JOB_REGS; ++i) {
            const int w = tid + i * (NW * 32);
            if (w < nword) reinterpret_cast<int*>(S.jobs_s)[w] = h.jw[i];
        }
        for (int w = tid + MMV_JOB_REGS * (NW * 32); w < nword; w += (NW * 32)) reinterpret_cast<int*>(S.jobs_s)[w] = reinterpret_cast<const int*>(p.jobs)[w];
        njobs = min(h.njobs, p.njobs_max);
        __syncthreads();
    }
    stamp();
    MatDesc m;
    m.W = p.W; m.expert_stride = p.expert_stride; m.e_base = p.e_base; m.Wsh = p.Wsh; m.E = p.E; m.jobs = MOE ? S.jobs_s : nullptr; m.jobw = nullptr; m.jobw0 = 0;
    m.rows = p.rows; m.K = p.K; m.out = p.out; m.ldo = p.ldo; m.accumulate = p.accumulate;
    const int upj = p.rows / 16;
    const unsigned total = (unsigned) njobs * upj;   // < 2^24: the products below stay inside 32 bits
    const int u0 = (int) (total * bid / nblk), u1 = (int) (total * (bid + 1) / nblk);
    const float* norm_w = MODE == MAT_DOWN ? nullptr : p.norm_w;
    bool ok = true, first = true;
    for (int uc = u0; uc < u1;) {
        const int j0 = uc / upj, j1 = min(j0 + JMAX, (u1 - 1) / upj + 1), ue = min(u1, j1 * upj);
        // the pass's first tile blocks are on their way while the rows are quantised
        if (!ring.pre) mat_preissue<MODE>(m, uc, ue, ring, warp, NW, lane, 2);
        // live rows: the dense rows [0, T), or the rows of the pass's jobs; the others are cleared
        int nlive = MOE ? 0 : p.T, cum[JMAX + 1];
        cum[0] = 0;
        if (MOE) {
#pragma unroll
            for (int sl = 0; sl < JMAX; ++sl) {
                const int n = j0 + sl < j1 ? min(S.jobs_s[j0 + sl].n, 4) : 0;
                cum[sl + 1] = cum[sl] + n;
            }
            nlive = cum[JMAX];
        }
        const bool given = !MOE && p.ximg;   // the image comes ready-made
        if (given) {
            const int n16 = (int) (stage_image_bytes(NG, p.K) / 16);
            float4* dst = reinterpret_cast<float4*>(S.cells);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = tid + j * (NW * 32);
                const float* d = j < 4 ? &h.v[j >> 1][(j & 1) * 4] : &h.w[(j - 4) >> 1][(j & 1) * 4];
                if (i < n16) dst[i] = make_float4(d[0], d[1], d[2], d[3]);
            }
            for (int i = tid + 8 * (NW * 32); i < n16; i += NW * 32) dst[i] = __ldcg(reinterpret_cast<const float4*>(p.ximg) + i);
        }
        const int ntask = given ? 0 : nlive * KB;
        for (int id0 = warp; id0 < ntask; id0 += NW * QUANT_BATCH) {
            QuantTask q[QUANT_BATCH];
#pragma unroll
            for (int j = 0; j < QUANT_BATCH; ++j) {
                const int id = id0 + j * NW;
                if (!MOE) q[j] = stage_dense_task(p, id);
                else {
                    q[j].src = nullptr;
                    q[j].t = q[j].blk = 0;
                    if (id < ntask) {
                        const int i = id % nlive;
                        int sl = 0;
#pragma unroll
                        for (int k = 1; k < JMAX; ++k) sl += i >= cum[k];
                        const int r = i - cum[sl];
                        const fnx_job& jb = S.jobs_s[j0 + sl];
                        q[j].t = sl * 4 + r;
                        q[j].blk = id / nlive;
                        q[j].src = p.x + (size_t) (MODE == MAT_DOWN ? jb.out[r] : jb.y[r]) * p.ldx + q[j].blk * 256;
                    }
                }
                if (MOE || !first || id0 != warp) {
                    quant_fetch(q[j], norm_w, lane, h.v[j], h.w[j]);
                    if (!MOE && q[j].src) post(q[j].t, q[j].blk, lane, h.v[j]);
                }
            }
            quant_finish(q, h.v, h.w, p.K, norm_w, S.cells, S.scales, S.rs, lane);
        }
        {   // the rows that hold nothing
            constexpr int TPR = (NW * 32) / NROW;   // threads per image row
            const int t = tid / TPR;
            bool live;
            if (!MOE) live = t < p.T;
            else live = j0 + t / 4 < j1 && (t & 3) < cum[t / 4 + 1] - cum[t / 4];
            const bool used = !MOE || j0 + t / 4 < j1;
            if (t < NROW && used && !live && !given) quant_zero_row(t, p.K, S.cells, S.scales, S.rs, tid % TPR, TPR);
        }
        first = false;
        __syncthreads();
        stamp();
        auto lane_x = [&](int j, LaneX<NG>& lx, int& ntok, int (&orow)[4 * NG]) {
            const int slot = MOE ? j - j0 : 0;
            if (!MOE) {
                ntok = p.T;
#pragma unroll
                for (int i = 0; i < 4 * NG; ++i) orow[i] = i;
            } else {
                const fnx_job& jb = S.jobs_s[j];
                ntok = min(jb.n, 4);
#pragma unroll
                for (int i = 0; i < 4 * NG; ++i) orow[i] = jb.out[i & 3];
            }
            lx = lane_x_dense<NG>(S.cells + (size_t) slot * NG * (p.K / 32) * 32, S.scales + (size_t) slot * NG * KB * 8, p.K, 4 * NG, lane);
            if (norm_w) {
                const int q = lane & 3;
#pragma unroll
                for (int ng = 0; ng < NG; ++ng) {
                    lx.r0[ng] = quant_row_factor(S.rs, slot * 4 * NG + 4 * ng + ((2 * q) & 3), p.K, p.eps);
                    lx.r1[ng] = quant_row_factor(S.rs, slot * 4 * NG + 4 * ng + ((2 * q + 1) & 3), p.K, p.eps);
                }
            }
        };
        if (ok) {
            ok = mat_items<NG, MODE>(m, uc, ue, S.table_s, ring, static_cast<PieceSlotT<NG, MODE>*>(S.pieces), warp, NW, lane, lane_x);
            if (!ok) atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
        }
        __syncthreads();
        stamp();
        if (ok) mat_combine<NG, MODE>(m, static_cast<const PieceSlotT<NG, MODE>*>(S.pieces), warp, NW, lane);
        uc = ue;
        if (uc < u1) __syncthreads();   // the images and the pieces are rewritten by the next pass
        stamp();
    }
    ring.pre = 0;
}

}  // namespace fnxb
