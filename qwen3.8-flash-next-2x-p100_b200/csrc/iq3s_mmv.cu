// IQ3_S matrix x few activation rows: the one kernel behind the dense projections (q/k/v/o, qkvz, ssm_out, head,
// MTP fc) and the routed/shared experts (gate|up + SwiGLU, down).
//
// Replaces the reference's decode-path quantised GEMVs: k_mmvq (engine/src/kernels.cu:192-228), k_q8s
// (engine/src/dense.cuh:211), k_moe_gu / k_moe_down (engine/src/moe.cuh:572-658) and the P100 lane-per-row
// kernel k_moe_rows (engine/src/p100_moe_rows.cuh:266-342).  Like the reference it multiplies integer codebook
// magnitudes by int8 activations and applies the scales afterwards; unlike it
//   - the weight stream is staged through shared memory by bulk async copies of 1,760-byte tile blocks, each warp
//     running its own ring of them (mmv_core.cuh), from the tile layout of iq3s_tile.h;
//   - the codebook lives in shared memory 32 times, once per bank, so the 9-bit lookups never conflict;
//   - activations are quantised to two int8 levels per 256-column block (x ~ d (q1 + q2 / 256), error
//     <= amax / 65024), and both levels of up to 4 rows ride in the 8 columns of one mma.sync.m16n8k32.s8, so a
//     decoded weight fragment is used for every row at once and the result is fp16-class accurate;
//   - a warp owns a 16-row tile across all of K (gate|up: the gate tile and its up tile), so nothing in the loop is
//     block-wide: no barrier, no shared partial sums; one block per SM walks a contiguous range of such units.
//
// Per-weight work is what bounds this kernel (about 2 integer instructions per weight besides the loads): the
// byte stream itself is 110 bytes per 256 weights.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fnx_common.cuh"
#include "mmv_stage.cuh"

namespace fnxb {

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

template <int NG, int MODE>
__global__ void __launch_bounds__(MMV_THREADS, 1) k_iq3s_mmv(const MmvParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int JMAX = mmv_jmax<MODE>(), NROW = JMAX * 4 * NG;
    const int KB = p.K / 256, R = p.R;
    uint8_t* table = smem_raw;
    StageSmem S;
    S.table_s = smem_u32(table);
    S.slots = table + CORE_TABLE_BYTES;
    S.bars = reinterpret_cast<uint64_t*>(S.slots + (size_t) MMV_WARPS * R * TILE_BYTES);
    S.bar_stride = R;
    S.cells = reinterpret_cast<uint2*>(S.bars + MMV_WARPS * R);
    S.scales = reinterpret_cast<float*>(S.cells + (size_t) JMAX * NG * (p.K / 32) * 32);
    S.rs = S.scales + (size_t) JMAX * NG * KB * 8;
    S.pieces = S.rs + NROW * 16;
    S.jobs_s = reinterpret_cast<fnx_job*>(reinterpret_cast<uint8_t*>(S.pieces) + (size_t) MMV_WARPS * 2 * sizeof(PieceSlotT<NG, MODE>));
    unsigned long long* prof = g_mmv_prof ? g_mmv_prof + (size_t) blockIdx.x * MMV_PROF_SLOTS : nullptr;
    int nstamp = 0;
    MMV_STAMP();
    pdl_launch_dependents();
    pdl_wait();   // from here on: what earlier kernels of the stream wrote (activations, job lists)
    // the job list or the first rows are fetched while the codebook is replicated and the barriers are set up
    StageRegs h;
    stage_begin<NG, MODE, MMV_WARPS>(p, h, tid, RowPlain());
    core_fill_table(table, tid, MMV_THREADS);
    if (lane == 0) {
        for (int i = 0; i < R; ++i) mbar_init(&S.bars[warp * R + i], 1);
        fence_barrier_init();
    }
    __syncthreads();
    WarpRing ring;
    ring.parity = 0;
    stage_ring(ring, S, R, warp);
    stage_run<NG, MODE, MMV_WARPS>(p, S, ring, h, tid, blockIdx.x, gridDim.x, RowPlain(), [&]() { MMV_STAMP(); });
    if (prof && tid == 0) prof[0] = (unsigned long long) nstamp;
}

template <int NG, int MODE>
static int launch_mmv(const MmvParams& p0, cudaStream_t st) {
    MmvParams p = p0;
    p.R = 6;   // tile blocks in flight per warp: as many as the shared memory left by the codebook and the images holds
    constexpr size_t LIMIT = 227 * 1024;
    while (p.R > 2 && mmv_smem_bytes<NG, MODE>(p.K, p.R, p.njobs_max) > LIMIT) --p.R;
    const size_t smem = mmv_smem_bytes<NG, MODE>(p.K, p.R, p.njobs_max);
    if (smem > LIMIT) return fail(FNX_E_ARG, "iq3s_mmv: %d columns x %d rows need %zu bytes of shared memory", p.K, 4 * NG, smem);
    if (int rc = set_smem_limit((const void*) k_iq3s_mmv<NG, MODE>, (int) LIMIT)) return rc;
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

extern "C" int fnx_dense_rows(int cols) { return cols <= 2048 ? FNX_DENSE_ROWS : 8; }

extern "C" int fnx_dense(const void* W, int rows, int cols, const float* x, int ldx, int T, const float* norm_w, float eps, float* y,
                         int ldy, int accumulate, unsigned* err, fnx_stream st) {
    if (int rc = check_cols(cols)) return rc;
    FNX_REQUIRE(W && x && y && err, "fnx_dense: null pointer");
    FNX_REQUIRE(T >= 1 && T <= fnx_dense_rows(cols), "fnx_dense: %d rows per call (1..%d at %d columns)", T, fnx_dense_rows(cols), cols);
    FNX_REQUIRE(rows > 0 && rows % 16 == 0, "fnx_dense: %d output rows, not a multiple of 16", rows);
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
    return T <= 4 ? launch_mmv<1, MAT_DENSE>(p, as_stream(st)) : T <= 8 ? launch_mmv<2, MAT_DENSE>(p, as_stream(st)) : launch_mmv<3, MAT_DENSE>(p, as_stream(st));
}

extern "C" int fnx_moe_gate_up(const void* Wgu, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs,
                               const int* njobs, int njobs_max, const float* x, const float* norm_w, float eps, int H, int F, float* h,
                               unsigned* err, fnx_stream st) {
    if (int rc = check_cols(H)) return rc;
    FNX_REQUIRE(Wgu && jobs && njobs && x && h && err, "fnx_moe_gate_up: null pointer");
    FNX_REQUIRE(F % 16 == 0, "fnx_moe_gate_up: ffn %d is not a multiple of 16", F);
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
    return launch_mmv<1, MAT_GATEUP>(p, as_stream(st));
}

extern "C" int fnx_moe_down(const void* Wdn, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs, const int* njobs,
                            int njobs_max, const float* h, int H, int F, float* part, unsigned* err, fnx_stream st) {
    if (int rc = check_cols(F)) return rc;
    FNX_REQUIRE(Wdn && jobs && njobs && h && part && err, "fnx_moe_down: null pointer");
    FNX_REQUIRE(H % 16 == 0, "fnx_moe_down: hidden %d is not a multiple of 16", H);
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
    return launch_mmv<1, MAT_DOWN>(p, as_stream(st));
}

extern "C" size_t fnx_dense_image_bytes(int cols) { return stage_image_bytes(FNX_DENSE_ROWS / 4, cols); }

extern "C" int fnx_dense_image(const void* W, int rows, int cols, const void* ximg, int T, int normed, float eps, float* y, int ldy, int accumulate,
                               unsigned* err, fnx_stream st) {
    if (int rc = check_cols(cols)) return rc;
    FNX_REQUIRE(W && ximg && y && err, "fnx_dense_image: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_DENSE_ROWS && cols <= 2048, "fnx_dense_image: %d rows per call (1..%d), %d columns (up to 2048)", T, FNX_DENSE_ROWS, cols);
    FNX_REQUIRE(rows > 0 && rows % 16 == 0, "fnx_dense_image: %d output rows, not a multiple of 16", rows);
    FNX_REQUIRE(((uintptr_t) ximg & 15) == 0 && ((uintptr_t) W & 15) == 0, "fnx_dense_image: the image and W must be 16-byte aligned");
    MmvParams p{};
    p.W = (const uint8_t*) W;
    p.T = T;
    p.ximg = (const uint8_t*) ximg;
    p.norm_w = normed ? (const float*) ximg : nullptr;   // only its presence matters: the image holds the normed rows' codes
    p.eps = eps;
    p.out = y;
    p.ldo = ldy;
    p.rows = rows;
    p.K = cols;
    p.accumulate = accumulate;
    p.err = err;
    return T <= 4 ? launch_mmv<1, MAT_DENSE>(p, as_stream(st)) : T <= 8 ? launch_mmv<2, MAT_DENSE>(p, as_stream(st)) : launch_mmv<3, MAT_DENSE>(p, as_stream(st));
}
