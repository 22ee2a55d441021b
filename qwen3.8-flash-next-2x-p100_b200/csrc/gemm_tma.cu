// Prompt-sized dense products from f16 operands in global memory: y[t][f] (+)= scale * sum_k W[f][k] x[t][k], on tcgen05.mma with
// both operands fetched by tensor copies.  Used by the prompt pass for the matrices that every row meets (input and output
// projections, decoded to f16 once per layer: moe_prefill.cu's k_pf_decode_f16; the router, whose f32 weights and rows are
// split into f16 high and low parts: three products restore the f32 operands; the tensor core adds into its f32 accumulator by
// truncation, ~2^-24 of the running sum a step, so the logits come out to a few 1e-5).  The counterpart of the reference's
// library GEMMs for prompts (cublasGemmEx, engine/src/prefill.cu:543-549, 626-629, 678-689; cublasSgemm for the router, :653).
//
// One block = NA x 128 features (tensor-memory lanes, NA accumulators) x 256 rows (columns); K in stages of 64 columns:
// boxes of 64 x 128 (weights) and 64 x 256 (rows) with the 128-byte swizzle, which is the layout the products' shared-memory
// descriptors name.  Warp 0: the loader thread; warp 1: the thread that issues the products; warps 2-5: the epilogue, a
// feature per thread, 32 rows at a time, so that a warp's stores cover 32 consecutive features of one row.  Tensor copies
// fill rows and features past the matrices' ends with zeros.  Every wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>

#include "fnx_common.cuh"

namespace fnxb {

constexpr int GT_M = 128;          // features per accumulator
constexpr int GT_N = 256;          // rows per block
constexpr int GT_KC = 64;          // K per stage: one 128-byte swizzle row
constexpr int GT_THREADS = 192;
constexpr int GT_A_BYTES = GT_M * GT_KC * 2;   // 16 KB: a box of weights
constexpr int GT_B_BYTES = GT_N * GT_KC * 2;   // 32 KB: a box of rows
constexpr unsigned GT_WAIT = 20000000u;

template <int NA, int NPROD>
struct GtShape {
    static constexpr int PARTS = NPROD == 3 ? 2 : 1;                          // high and low parts of each operand
    static constexpr int STAGE = PARTS * (NA * GT_A_BYTES + GT_B_BYTES);
    static constexpr int STAGES = (220 * 1024) / STAGE < 4 ? (220 * 1024) / STAGE : 4;
    static constexpr int SMEM = 1024 + STAGES * STAGE + 256;
};

struct GtParams {
    float* y;
    int ldy, T, rows, K, accumulate;
    float scale;
    unsigned* err;
};

__device__ __forceinline__ uint64_t gt_desc(uint32_t saddr) {
    // K-major tile with the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart (layout type 2, version 1)
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) 1 << 16) | ((uint64_t) (1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gt_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void gt_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void gt_tma_2d(uint32_t dst_s, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_s), "l"(map), "r"(c0),
                 "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void gt_ld32(uint32_t taddr, float (&v)[32]) {
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

// grid (feature tiles of NA x 128, row tiles of 256): the feature tiles of one row tile run together, so the rows' boxes are
// shared through L2 and the weights stay there from one row tile to the next.
// map_w / map_x: the operands (NPROD = 3: their high parts), map_wl / map_xl: the low parts.
template <int NA, int NPROD>
__global__ void __launch_bounds__(GT_THREADS, 1) k_gemm_tma(const GtParams p, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                           const __grid_constant__ CUtensorMap map_wl, const __grid_constant__ CUtensorMap map_xl) {
    using Sh = GtShape<NA, NPROD>;
    constexpr int STAGES = Sh::STAGES, PARTS = Sh::PARTS;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Sh::STAGE);   // a stage's boxes have landed
    uint64_t* empty = full + STAGES;                                           // a stage's products have finished
    uint64_t* done = empty + STAGES;                                           // every product has finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int f0 = blockIdx.x * NA * GT_M, t0 = blockIdx.y * GT_N, nk = p.K / GT_KC;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(done, 1);
        fence_barrier_init();
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NA * GT_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // a stage: [weights (high)] [weights low] [rows (high)] [rows low]
    auto a_of = [&](int s, int part) { return smem + s * Sh::STAGE + part * NA * GT_A_BYTES; };
    auto b_of = [&](int s, int part) { return smem + s * Sh::STAGE + PARTS * NA * GT_A_BYTES + part * GT_B_BYTES; };
    if (tid == 0) {
        for (int kb = 0; kb < nk; ++kb) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait_bounded(&empty[s], (unsigned) ((kb / STAGES - 1) & 1), GT_WAIT)) {
                atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
                break;
            }
            mbar_expect_tx(&full[s], (unsigned) Sh::STAGE);
#pragma unroll
            for (int part = 0; part < PARTS; ++part) {
#pragma unroll
                for (int a = 0; a < NA; ++a) gt_tma_2d(smem_u32(a_of(s, part) + a * GT_A_BYTES), part ? &map_wl : &map_w, kb * GT_KC, f0 + a * GT_M, &full[s]);
                gt_tma_2d(smem_u32(b_of(s, part)), part ? &map_xl : &map_x, kb * GT_KC, t0, &full[s]);
            }
        }
    } else if (tid == 32) {
        // f32 accumulate, f16 x f16, both operands K-major, N = 256, M = 128
        constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (GT_N >> 3) << 17) | ((uint32_t) (GT_M >> 4) << 24);
        bool ok = true;
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % STAGES;
            ok = mbar_wait_bounded(&full[s], (unsigned) ((kb / STAGES) & 1), GT_WAIT);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k16 = 0; k16 < GT_KC / 16; ++k16) {
#pragma unroll
                for (int a = 0; a < NA; ++a) {
                    const uint32_t d = tmem + a * GT_N;
                    const uint64_t ah = gt_desc(smem_u32(a_of(s, 0) + a * GT_A_BYTES) + k16 * 32), bh = gt_desc(smem_u32(b_of(s, 0)) + k16 * 32);
                    gt_mma(d, ah, bh, IDESC, (kb | k16) != 0);
                    if (NPROD == 3) {
                        const uint64_t al = gt_desc(smem_u32(a_of(s, 1) + a * GT_A_BYTES) + k16 * 32), bl = gt_desc(smem_u32(b_of(s, 1)) + k16 * 32);
                        gt_mma(d, ah, bl, IDESC, 1);
                        gt_mma(d, al, bh, IDESC, 1);
                    }
                }
            }
            gt_commit(&empty[s]);
        }
        if (ok) gt_commit(done);
        else atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
    } else if (warp >= 2) {
        // the epilogue: warp w reads lanes 32 (w % 4) .. + 31: a feature per thread
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(done, 0u, GT_WAIT));
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int lg = warp & 3;
#pragma unroll 1
            for (int a = 0; a < NA; ++a) {
                const int f = f0 + a * GT_M + 32 * lg + lane;
#pragma unroll 1
                for (int c = 0; c < GT_N / 32; ++c) {
                    if (t0 + c * 32 >= p.T) break;
                    float v[32];
                    gt_ld32(tmem + ((uint32_t) (32 * lg) << 16) + (uint32_t) (a * GT_N + c * 32), v);
                    if (f < p.rows) {
                        float* o = p.y + (size_t) (t0 + c * 32) * p.ldy + f;
                        const int nt = min(32, p.T - (t0 + c * 32));
                        float old[32];
                        if (p.accumulate) {   // every load first: the stores below would otherwise order them one by one
#pragma unroll
                            for (int i = 0; i < 32; ++i) old[i] = i < nt ? __ldcs(o + (size_t) i * p.ldy) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < nt) __stcs(o + (size_t) i * p.ldy, p.accumulate ? old[i] + v[i] * p.scale : v[i] * p.scale);
                    }
                }
            }
        } else if (lane == 0) {
            atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NA * GT_N) : "memory");
}

// ---- the grouped expert products of a prompt from f16 weights (every expert's matrix decoded once per layer, expert e at
// rows [e R, (e + 1) R) of one stacked matrix) and rows laid out in job order (x_sorted / h_sorted: entry `pos` of the job
// list's `order`), so that both operands of a job's tile are boxes of the same two tensors.  A job is up to 256 consecutive
// entries of one expert; the rows of a tile past the job's end are computed and dropped.
//   MODE 1: gate|up with SwiGLU: accumulator 0 = 128 gate features, accumulator 1 = the same up features; h = silu(g) u as f16
//           into h_sorted [pos][F].
//   MODE 0: down: 256 features; part[pair][f] f32 at the pair index order[pos].
struct GtJob {
    int w, n, start;   // expert (E: the shared expert), rows, first entry of `order`
};
struct GtJobParams {
    const GtJob* jobs;
    const int* njobs;
    const int* order;
    int R;             // feature rows of one expert in the stacked weight matrix (gate|up: 2 F; down: H)
    int F;             // MODE 1: the ffn width (gate rows [0, F), up rows [F, 2 F))
    int K;
    __half* h_sorted;  // MODE 1
    float* part;       // MODE 0
    int H;             // MODE 0: floats per row of part
    unsigned* err;
};

template <int MODE>
__global__ void __launch_bounds__(GT_THREADS, 1) k_gemm_tma_jobs(const GtJobParams p, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x) {
    using Sh = GtShape<2, 1>;
    constexpr int STAGES = Sh::STAGES, NA = 2;
    const int j = blockIdx.y;
    if (j >= *p.njobs) return;
    const GtJob job = p.jobs[j];
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Sh::STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* done = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = p.K / GT_KC;
    // the two weight boxes of the block: gate and up rows of the same 128 features, or 256 consecutive features
    const int f0 = MODE == 1 ? blockIdx.x * GT_M : blockIdx.x * NA * GT_M;
    const int wrow0 = job.w * p.R + f0, wrow1 = MODE == 1 ? wrow0 + p.F : wrow0 + GT_M;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(done, 1);
        fence_barrier_init();
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NA * GT_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    auto a_of = [&](int s, int a) { return smem + s * Sh::STAGE + a * GT_A_BYTES; };
    auto b_of = [&](int s) { return smem + s * Sh::STAGE + NA * GT_A_BYTES; };
    if (tid == 0) {
        for (int kb = 0; kb < nk; ++kb) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait_bounded(&empty[s], (unsigned) ((kb / STAGES - 1) & 1), GT_WAIT)) {
                atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
                break;
            }
            mbar_expect_tx(&full[s], (unsigned) Sh::STAGE);
            gt_tma_2d(smem_u32(a_of(s, 0)), &map_w, kb * GT_KC, wrow0, &full[s]);
            gt_tma_2d(smem_u32(a_of(s, 1)), &map_w, kb * GT_KC, wrow1, &full[s]);
            gt_tma_2d(smem_u32(b_of(s)), &map_x, kb * GT_KC, job.start, &full[s]);
        }
    } else if (tid == 32) {
        constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (GT_N >> 3) << 17) | ((uint32_t) (GT_M >> 4) << 24);
        bool ok = true;
        for (int kb = 0; kb < nk && ok; ++kb) {
            const int s = kb % STAGES;
            ok = mbar_wait_bounded(&full[s], (unsigned) ((kb / STAGES) & 1), GT_WAIT);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k16 = 0; k16 < GT_KC / 16; ++k16) {
                const uint64_t bd = gt_desc(smem_u32(b_of(s)) + k16 * 32);
#pragma unroll
                for (int a = 0; a < NA; ++a) gt_mma(tmem + a * GT_N, gt_desc(smem_u32(a_of(s, a)) + k16 * 32), bd, IDESC, (kb | k16) != 0);
            }
            gt_commit(&empty[s]);
        }
        if (ok) gt_commit(done);
        else atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
    } else if (warp >= 2) {
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(done, 0u, GT_WAIT));
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int lg = warp & 3;
            const uint32_t lane_base = (uint32_t) (32 * lg) << 16;
            if (MODE == 1) {
                const int f = f0 + 32 * lg + lane;
#pragma unroll 1
                for (int c = 0; c < GT_N / 32; ++c) {
                    if (c * 32 >= job.n) break;
                    float g[32], u[32];
                    gt_ld32(tmem + lane_base + (uint32_t) (c * 32), g);
                    gt_ld32(tmem + lane_base + (uint32_t) (GT_N + c * 32), u);
                    __half* o = p.h_sorted + (size_t) (job.start + c * 32) * p.F + f;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < job.n) o[(size_t) i * p.F] = __float2half_rn(siluf_(g[i]) * u[i]);
                }
            } else {
#pragma unroll 1
                for (int a = 0; a < NA; ++a) {
                    const int f = f0 + a * GT_M + 32 * lg + lane;
#pragma unroll 1
                    for (int c = 0; c < GT_N / 32; ++c) {
                        if (c * 32 >= job.n) break;
                        float v[32];
                        gt_ld32(tmem + lane_base + (uint32_t) (a * GT_N + c * 32), v);
                        const int my = c * 32 + lane < job.n ? p.order[job.start + c * 32 + lane] : 0;   // the chunk's pair indices, one per lane
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int pair = __shfl_sync(0xffffffffu, my, i);
                            if (c * 32 + i < job.n) __stcs(p.part + (size_t) pair * p.H + f, v[i]);
                        }
                    }
                }
            }
        } else if (lane == 0) {
            atomicOr(p.err, (unsigned) FNX_ERR_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NA * GT_N) : "memory");
}

// an f16 matrix [rows][K] as a rank-2 tensor for boxes of 64 columns x box_rows rows with the 128-byte swizzle
static int gt_map(CUtensorMap* map, const __half* base, int rows, int K, int box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        FNX_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(FNX_E_UNAVAILABLE, "the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeFn) fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t) K, (cuuint64_t) rows};
    const cuuint64_t strides[1] = {(cuuint64_t) K * 2};
    const cuuint32_t box[2] = {(cuuint32_t) GT_KC, (cuuint32_t) box_rows}, estr[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*) base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(FNX_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int) rc);
    return FNX_OK;
}

// y[t][f] (+)= scale * W[f] . x[t] over T rows and `rows` features; wl / xl: the operands' low parts (null: one product)
int gemm_tma_launch(const __half* w, const __half* wl, const __half* x, const __half* xl, float* y, int ldy, int T, int rows, int K, int accumulate, float scale,
                    unsigned* err, cudaStream_t st) {
    FNX_REQUIRE(w && x && y && err && T >= 1 && rows >= 1 && K >= GT_KC && K % GT_KC == 0, "gemm_tma: %d rows x %d features x %d", T, rows, K);
    FNX_REQUIRE((((uintptr_t) w | (uintptr_t) x | (uintptr_t) wl | (uintptr_t) xl) & 15) == 0, "gemm_tma: operands must be 16-byte aligned");
    FNX_REQUIRE((wl == nullptr) == (xl == nullptr), "gemm_tma: low parts of both operands or of neither");
    GtParams p{y, ldy, T, rows, K, accumulate, scale, err};
    CUtensorMap mw, mx, mwl, mxl;
    FNX_TRY(gt_map(&mw, w, rows, K, GT_M));
    FNX_TRY(gt_map(&mx, x, T, K, GT_N));
    if (wl) {
        FNX_TRY(gt_map(&mwl, wl, rows, K, GT_M));
        FNX_TRY(gt_map(&mxl, xl, T, K, GT_N));
        using Sh = GtShape<1, 3>;
        if (int rc = set_smem_limit((const void*) k_gemm_tma<1, 3>, Sh::SMEM)) return rc;
        k_gemm_tma<1, 3><<<dim3((rows + GT_M - 1) / GT_M, (T + GT_N - 1) / GT_N), GT_THREADS, Sh::SMEM, st>>>(p, mw, mx, mwl, mxl);
    } else {
        mwl = mw;
        mxl = mx;
        using Sh = GtShape<2, 1>;
        if (int rc = set_smem_limit((const void*) k_gemm_tma<2, 1>, Sh::SMEM)) return rc;
        k_gemm_tma<2, 1><<<dim3((rows + 2 * GT_M - 1) / (2 * GT_M), (T + GT_N - 1) / GT_N), GT_THREADS, Sh::SMEM, st>>>(p, mw, mx, mwl, mxl);
    }
    FNX_LAUNCH_OK("k_gemm_tma");
    return FNX_OK;
}

// the two grouped products of a layer's experts: h_sorted = silu(gate) up over x_sorted, then part = down over h_sorted.
// gu16 [(experts + 1)][2 F][H], dn16 [(experts + 1)][H][F] (the last slot: the shared expert); entries = rows of x_sorted.
int gemm_tma_experts(const __half* gu16, const __half* dn16, int slots, const __half* x_sorted, __half* h_sorted, float* part, const void* jobs, const int* njobs,
                     const int* order, int max_jobs, int entries, int H, int F, unsigned* err, cudaStream_t st) {
    using Sh = GtShape<2, 1>;
    if (int rc = set_smem_limit((const void*) k_gemm_tma_jobs<1>, Sh::SMEM)) return rc;
    if (int rc = set_smem_limit((const void*) k_gemm_tma_jobs<0>, Sh::SMEM)) return rc;
    CUtensorMap mw, mx;
    GtJobParams p{};
    p.jobs = (const GtJob*) jobs; p.njobs = njobs; p.order = order; p.err = err;
    FNX_TRY(gt_map(&mw, gu16, slots * 2 * F, H, GT_M));
    FNX_TRY(gt_map(&mx, x_sorted, entries, H, GT_N));
    p.R = 2 * F; p.F = F; p.K = H; p.h_sorted = h_sorted;
    k_gemm_tma_jobs<1><<<dim3(F / GT_M, max_jobs), GT_THREADS, Sh::SMEM, st>>>(p, mw, mx);
    FNX_LAUNCH_OK("k_gemm_tma_jobs (gate|up)");
    FNX_TRY(gt_map(&mw, dn16, slots * H, F, GT_M));
    FNX_TRY(gt_map(&mx, h_sorted, entries, F, GT_N));
    p.R = H; p.K = F; p.part = part; p.H = H; p.h_sorted = nullptr;
    k_gemm_tma_jobs<0><<<dim3(H / (2 * GT_M), max_jobs), GT_THREADS, Sh::SMEM, st>>>(p, mw, mx);
    FNX_LAUNCH_OK("k_gemm_tma_jobs (down)");
    return FNX_OK;
}

}  // namespace fnxb
